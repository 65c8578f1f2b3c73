"""GPU parity of the attention core and of the whole sageattn call.

Tolerance (stated by the task): cosine similarity >= 0.9995 and max-abs error <= 2e-2 in the
output dtype's range, against (a) the CPU oracle fed the same int8 tensors and scales and
(b) the reference's sm80 CUDA kernel rebuilt for sm_100 (oracle/_ref) on the same inputs.
"""
import pytest
import torch

from gpu_util import cuda_or_fail, make_qkv, reference_ops
from oracle import sage_oracle as O

pytestmark = pytest.mark.gpu

COS_MIN = 0.9995
MAX_ABS = 2e-2
CFG = (128, 64, 32, 64)


def _run_core(q, k, v, layout, causal, mode, gran="per_thread", sm_scale=None, return_lse=False, smooth=True):
    from sageattention import quant
    from sageattention.core import attn_fwd_quantized
    km = quant.mean_k(k, layout) if smooth else None
    if gran == "per_thread":
        q8, qs, k8, ks = quant.per_thread_int8(q, k, km, *[CFG[i] for i in (0, 2, 1, 3)], layout, div="ieee")
    else:
        q8, qs, k8, ks = quant.per_block_int8(q, k, km, 128, 64, layout, div="ieee")
    v16 = quant.cast_v_fp16(v, layout)
    out = torch.empty_like(q)
    sc = sm_scale if sm_scale is not None else q.size(-1) ** -0.5
    lse = attn_fwd_quantized(q8, k8, v16, out, qs, ks, layout, causal, sc, CFG, mode, return_lse, gran)
    torch.cuda.synchronize()
    return out, lse, (q8, qs, k8, ks, v16)


def _oracle(quantised, layout, causal, mode, gran, dtype, sm_scale=None):
    q8, qs, k8, ks, v16 = [t.cpu() for t in quantised]
    return O.attend(q8, k8, v16, qs, ks, layout, causal, sm_scale, mode, gran, 128, 32, 64, 64, dtype, True)


def _assert_close(got, exp, what, max_abs=MAX_ABS, rounded_sum=False):
    """cos >= 0.9995 and max-abs <= 2e-2.  For bf16 outputs one unit in the last place is 0.03125
    once |o| >= 4 (early causal rows see few keys and reach such values), so there the bound is
    one bf16 ulp of the expected value: a single rounding flip, nothing more.  `rounded_sum`: the
    output is a bf16 sum of the attention result and a larger term (the V mean), so two results that
    differ by up to `max_abs` before that last rounding may land one more grid step apart."""
    got, exp = got.cpu(), exp.cpu()
    c = O.compare(got, exp)
    bound = torch.full_like(exp.float(), max_abs)
    if exp.dtype == torch.bfloat16:
        ulp = torch.exp2(torch.floor(torch.log2(exp.float().abs().clamp_min(1e-30))) - 7)
        bound = (bound + ulp) if rounded_sum else torch.maximum(bound, ulp)
    worst = float(((got.float() - exp.float()).abs() - bound).max())
    assert c["cos"] >= COS_MIN and worst <= 0.0, (what, c, worst)
    return c


@pytest.mark.parametrize("mode", ["fp32", "fp16+fp32", "fp16"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D,dtype,layout", [(128, torch.float16, "HND"), (64, torch.float16, "NHD"),
                                             (128, torch.bfloat16, "NHD")])
def test_core_matches_oracle(D, dtype, layout, causal, mode):
    cuda_or_fail()
    q, k, v = make_qkv(1, 4, 2, 512, D, dtype, layout, seed=11, k_bias=1.0)
    out, lse, qz = _run_core(q, k, v, layout, causal, mode, return_lse=True)
    exp, exp_lse = _oracle(qz, layout, causal, mode, "per_thread", dtype)
    _assert_close(out, exp, (D, dtype, layout, causal, mode))
    assert float((lse.cpu() - exp_lse).abs().max()) <= 2e-2


@pytest.mark.parametrize("N,Nkv", [(1, 1), (63, 63), (129, 129), (200, 200), (256, 256), (257, 257), (300, 1000),
                                   (1000, 300), (777, 777)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("mode,D", [("fp32", 128), ("fp16+fp32", 128), ("fp16+fp32", 64), ("fp16", 256)])
def test_core_ragged_lengths(N, Nkv, causal, mode, D):
    """Lengths from one row to several blocks, query and key lengths that differ, on both kernels
    (one and two query tiles per CTA) and the head_dim 256 configuration; output and LSE."""
    cuda_or_fail()
    q, k, v = make_qkv(2, 2, 2, N, D, torch.float16, "HND", seed=N + Nkv, Nkv=Nkv, k_bias=0.5)
    out, lse, qz = _run_core(q, k, v, "HND", causal, mode, return_lse=True)
    exp, exp_lse = _oracle(qz, "HND", causal, mode, "per_thread", torch.float16)
    _assert_close(out, exp, (N, Nkv, causal, mode, D))
    assert float((lse.cpu() - exp_lse).abs().max()) <= 2e-2


def test_core_per_block_config1():
    """The tiny correctness case: B=1, H=2, N=256, D=64, fp16, NHD, non-causal, smooth_k, fp32, per-block 128/64."""
    cuda_or_fail()
    q, k, v = make_qkv(1, 2, 2, 256, 64, torch.float16, "NHD", seed=0)
    out, _, qz = _run_core(q, k, v, "NHD", False, "fp32", gran="per_block")
    exp, _ = _oracle(qz, "NHD", False, "fp32", "per_block", torch.float16)
    _assert_close(out, exp, "config1")
    # the quantiser is bit-exact given the same K mean: feed the oracle the mean the GPU computed
    from sageattention import quant
    q8, qs, k8, ks = O.quant_per_block(q.cpu(), k.cpu(), quant.mean_k(k, "NHD").cpu(), 128, 64, "NHD")
    assert torch.equal(qz[0].cpu(), q8) and torch.equal(qz[2].cpu(), k8)
    assert torch.equal(qz[1].cpu(), qs) and torch.equal(qz[3].cpu(), ks)


def test_core_sm_scale_argument():
    cuda_or_fail()
    q, k, v = make_qkv(1, 2, 2, 384, 128, torch.float16, "HND", seed=3)
    out, _, qz = _run_core(q, k, v, "HND", False, "fp32", sm_scale=0.05)
    exp, _ = _oracle(qz, "HND", False, "fp32", "per_thread", torch.float16, sm_scale=0.05)
    _assert_close(out, exp, "sm_scale")


@pytest.mark.parametrize("mode,op", [("fp32", "qk_int8_sv_f16_accum_f32_attn"),
                                      ("fp16+fp32", "qk_int8_sv_f16_accum_f16_attn_inst_buf"),
                                      ("fp16", "qk_int8_sv_f16_accum_f16_attn")])
@pytest.mark.parametrize("case", ["c2_like", "c3_like", "c4_like", "c5_like", "d256"])
def test_core_matches_reference_cuda_kernel(case, mode, op):
    """Same int8 tensors and scales into the reference's sm80 kernel (rebuilt for sm_100) and ours."""
    cuda_or_fail()
    ref = reference_ops()
    assert ref is not None, "oracle/_ref/libsage_ref_sm80.so is missing: run make -C oracle"
    if case == "c2_like":     # SD-style: D=64 fp16 HND, K offset N(0, 3^2)
        args = dict(B=2, Hq=4, Hkv=4, N=1024, D=64, dtype=torch.float16, layout="HND", seed=1, k_bias=3.0)
        causal = False
    elif case == "c3_like":   # GQA prefill: D=128 bf16 NHD causal, 4 outlier channels x20
        args = dict(B=1, Hq=8, Hkv=2, N=2048, D=128, dtype=torch.bfloat16, layout="NHD", seed=2, k_outliers=20.0)
        causal = True
    elif case == "c4_like":   # video DiT: ragged length, bf16 HND, K bias N(0, 2^2)
        args = dict(B=1, Hq=2, Hkv=2, N=2320, D=128, dtype=torch.bfloat16, layout="HND", seed=3, k_bias=2.0)
        causal = False
    elif case == "d256":      # head_dim 256 (one query tile per CTA): GQA, ragged length, causal
        args = dict(B=1, Hq=4, Hkv=2, N=1500, D=256, dtype=torch.bfloat16, layout="NHD", seed=5, k_bias=1.0)
        causal = True
    else:                     # long-context causal fp16
        args = dict(B=1, Hq=4, Hkv=4, N=4096, D=128, dtype=torch.float16, layout="HND", seed=4)
        causal = True
    q, k, v = make_qkv(**args)
    layout = args["layout"]
    out, _, (q8, qs, k8, ks, v16) = _run_core(q, k, v, layout, causal, mode)
    ref_out = torch.empty_like(q)
    getattr(ref, op)(q8, k8, v16, ref_out, qs, ks, 0 if layout == "NHD" else 1, causal,
                     q.size(-1) ** -0.5, *CFG, False)
    torch.cuda.synchronize()
    c = _assert_close(out, ref_out, (case, mode))
    print(case, mode, c)


@pytest.mark.parametrize("mode,op", [("fp32", "qk_int8_sv_f16_accum_f32_attn"),
                                      ("fp16+fp32", "qk_int8_sv_f16_accum_f16_attn_inst_buf"),
                                      ("fp16", "qk_int8_sv_f16_accum_f16_attn")])
@pytest.mark.parametrize("D,dtype,layout,N", [(128, torch.bfloat16, "HND", 2320), (64, torch.float16, "NHD", 1024),
                                              (256, torch.float16, "HND", 700)])
def test_32_key_scale_blocks_match_reference_cuda_kernel(D, dtype, layout, N, mode, op):
    """The reference's (BLKQ, BLKK, WARPQ, WARPK) = (128, 32, 32, 32) candidate: K scales per 32 keys
    (sixteen scale classes per 128-key block).  Non-causal against the reference kernel (it accepts this
    configuration for non-causal attention only), causal and non-causal against the oracle."""
    from sageattention import quant
    from sageattention.core import attn_fwd_quantized
    cuda_or_fail()
    ref = reference_ops()
    assert ref is not None, "oracle/_ref/libsage_ref_sm80.so is missing: run make -C oracle"
    cfg = (128, 32, 32, 32)
    q, k, v = make_qkv(1, 4, 2, N, D, dtype, layout, seed=71, k_bias=1.5)
    km = quant.mean_k(k, layout)
    q8, qs, k8, ks = quant.per_thread_int8(q, k, km, 128, 32, 32, 32, layout, div="ieee")
    v16 = quant.cast_v_fp16(v, layout)
    for causal in (False, True):
        out = torch.empty_like(q)
        lse = attn_fwd_quantized(q8, k8, v16, out, qs, ks, layout, causal, D ** -0.5, cfg, mode, True)
        torch.cuda.synchronize()
        exp, exp_lse = O.attend(q8.cpu(), k8.cpu(), v16.cpu(), qs.cpu(), ks.cpu(), layout, causal, None, mode,
                                "per_thread", 128, 32, 32, 32, dtype, True)
        _assert_close(out, exp, ("blk_k 32 vs oracle", D, causal, mode))
        assert float((lse.cpu() - exp_lse).abs().max()) <= 2e-2
        if not causal:
            ref_out = torch.empty_like(q)
            getattr(ref, op)(q8, k8, v16, ref_out, qs, ks, 0 if layout == "NHD" else 1, False, D ** -0.5, *cfg, False)
            torch.cuda.synchronize()
            _assert_close(out, ref_out, ("blk_k 32 vs reference", D, mode))
    # the per-block scheme with 32-key blocks, through the public call
    import sageattention
    from sageattention.core import _sageattn_configured
    o_blk = _sageattn_configured(q, k, v, layout, False, mode, True, False, False, cfg, None, "per_block")
    exp_blk, _ = O.sdpa_fp32(q.cpu(), k.cpu(), v.cpu(), layout, False)
    c = O.compare(o_blk.cpu(), exp_blk)
    assert c["fro_rel"] <= 0.02 and c["max_abs"] <= 0.1, c


@pytest.mark.parametrize("case", ["c2_like", "c3_like", "c4_like"])
def test_fuse_v_mean_matches_reference_cuda_kernel(case):
    """smooth_v: V minus its channel mean through the fp16 accumulator, the mean added back in the
    epilogue.  The smoothed V and the mean (ours: bit-identical to the torch expressions of the
    reference when fed the same mean) go into the reference's ..._fuse_v_mean_attn kernel and ours."""
    from sageattention import quant
    from sageattention.core import attn_fwd_quantized
    cuda_or_fail()
    ref = reference_ops()
    assert ref is not None, "oracle/_ref/libsage_ref_sm80.so is missing: run make -C oracle"
    if case == "c2_like":
        args = dict(B=2, Hq=4, Hkv=4, N=1024, D=64, dtype=torch.float16, layout="HND", seed=11, k_bias=3.0)
        causal = False
    elif case == "c3_like":
        args = dict(B=1, Hq=8, Hkv=2, N=2048, D=128, dtype=torch.bfloat16, layout="NHD", seed=12, k_outliers=20.0)
        causal = True
    else:
        args = dict(B=1, Hq=2, Hkv=2, N=2320, D=128, dtype=torch.bfloat16, layout="HND", seed=13, k_bias=2.0)
        causal = False
    q, k, v = make_qkv(**args)
    layout = args["layout"]
    seq_dim = 2 if layout == "HND" else 1
    v = v + 1.5 * torch.randn_like(v.select(seq_dim, 0)).unsqueeze(seq_dim)          # a channel offset worth removing
    v_s, vm = quant.smooth_v_fp16(v, layout)
    # the smoothing itself: exactly the reference's torch expression on the same mean, and the mean
    # within one unit in the last place of torch's
    assert torch.equal(v_s, (v - vm.unsqueeze(seq_dim)).to(torch.float16))
    vm_t = v.mean(dim=seq_dim)
    ulp = torch.exp2(torch.floor(torch.log2(vm_t.float().abs().clamp_min(1e-30))) - (10 if v.dtype == torch.float16 else 7))
    assert bool(((vm.float() - vm_t.float()).abs() <= ulp).all())
    km = quant.mean_k(k, layout)
    q8, qs, k8, ks = quant.per_thread_int8(q, k, km, *[CFG[i] for i in (0, 2, 1, 3)], layout, div="ieee")
    out = torch.empty_like(q)
    attn_fwd_quantized(q8, k8, v_s, out, qs, ks, layout, causal, q.size(-1) ** -0.5, CFG, "fp16", False,
                       "per_thread", None, vm)
    ref_out = torch.empty_like(q)
    ref.qk_int8_sv_f16_accum_f16_fuse_v_mean_attn(q8, k8, v_s, ref_out, qs, ks, vm, 0 if layout == "NHD" else 1, causal,
                                                  q.size(-1) ** -0.5, *CFG, False)
    torch.cuda.synchronize()
    _assert_close(out, ref_out, ("fuse_v_mean", case), rounded_sum=True)
    exp = O.attend(q8.cpu(), k8.cpu(), v_s.cpu(), qs.cpu(), ks.cpu(), layout, causal, None, "fp16", "per_thread",
                   128, 32, 64, 64, q.dtype, False, v_mean=vm.cpu())
    _assert_close(out, exp, ("fuse_v_mean vs oracle", case), rounded_sum=True)


def test_sageattn_smooth_v_front_end():
    """smooth_v=True through the public call: fp16 accumulate takes the smoothed path and stays within
    the reference's acceptance bounds against exact attention even with a large V offset, where the
    plain fp16 accumulator loses accuracy; the fp32 modes warn and ignore it as the reference does."""
    import warnings
    import sageattention
    cuda_or_fail()
    q, k, v = make_qkv(1, 4, 4, 2048, 128, torch.float16, "HND", seed=21)
    v = v + 8.0 * torch.randn(1, 4, 1, 128, device=v.device, dtype=v.dtype)
    exp, _ = O.sdpa_fp32(q.cpu(), k.cpu(), v.cpu(), "HND", True)
    out = sageattention.sageattn(q, k, v, is_causal=True, pv_accum_dtype="fp16", smooth_v=True)
    c = O.compare(out.cpu(), exp)
    assert c["fro_rel"] <= 0.02 and c["max_abs"] <= 0.1, c
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        out32 = sageattention.sageattn(q, k, v, is_causal=True, pv_accum_dtype="fp32", smooth_v=True)
    assert any("smooth_v will be ignored" in str(x.message) for x in w)
    assert torch.equal(out32, sageattention.sageattn(q, k, v, is_causal=True, pv_accum_dtype="fp32"))


@pytest.mark.parametrize("layout", ["HND", "NHD"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
def test_sageattn_end_to_end_vs_sdpa(layout, dtype, causal):
    """The reference's own acceptance test (tests/test_sageattn.py:52-61): fro-rel <= 0.02 and
    max-abs <= 0.1 against SDPA-math, here for every head_dim incl. a padded one."""
    import sageattention
    cuda_or_fail()
    for D in (64, 128, 80, 200, 256):
        q, k, v = make_qkv(2, 4, 4, 1024, D, dtype, layout, seed=D)
        for mode in ("fp32", "fp16+fp32", "fp16"):
            for smooth_k in (True, False):
                out = sageattention.sageattn(q, k, v, tensor_layout=layout, is_causal=causal,
                                             pv_accum_dtype=mode, smooth_k=smooth_k)
                exp, _ = O.sdpa_fp32(q.cpu(), k.cpu(), v.cpu(), layout, causal)
                c = O.compare(out.cpu(), exp)
                assert out.shape == q.shape and out.dtype == dtype
                assert c["fro_rel"] <= 0.02 and c["max_abs"] <= 0.1, (D, mode, smooth_k, c)


def test_sageattn_return_lse_gqa_causal():
    """The GQA prefill case in small: GQA, causal, bf16, NHD, outlier channels, return_lse.  The LSE
    (natural log, with the smooth-k correction added back) is checked against the CPU oracle run
    through the same pipeline, and loosely against exact attention (int8 error on outlier-heavy K
    dominates that distance)."""
    import sageattention
    cuda_or_fail()
    q, k, v = make_qkv(1, 8, 2, 1024, 128, torch.bfloat16, "NHD", seed=9, k_outliers=20.0)
    out, lse = sageattention.sageattn(q, k, v, tensor_layout="NHD", is_causal=True, return_lse=True)
    assert lse.shape == (1, 8, 1024) and lse.dtype == torch.float32
    o_exp, lse_exp = O.sageattn(q.cpu(), k.cpu(), v.cpu(), "NHD", True, "fp32", True, True)
    assert float((lse.cpu() - lse_exp).abs().max()) <= 2e-2
    _assert_close(out, o_exp, "c3 small vs oracle")
    exact, exact_lse = O.sdpa_fp32(q.cpu(), k.cpu(), v.cpu(), "NHD", True)
    assert float((lse.cpu() - exact_lse).abs().max()) <= 1.0
    assert O.compare(out.cpu(), exact)["fro_rel"] <= 0.1


def test_sageattn_linearity_in_v_at_full_size():
    """Size-independent property on a full-length head (N = 32768, D = 128, causal): the output is
    linear in V, and with V = const every row returns that constant."""
    import sageattention
    cuda_or_fail()
    q, k, v = make_qkv(1, 2, 2, 32768, 128, torch.float16, "HND", seed=4)
    ones = torch.full_like(v, 0.5)
    out = sageattention.sageattn(q, k, ones, is_causal=True, pv_accum_dtype="fp16+fp32")
    assert float((out.float() - 0.5).abs().max()) <= 2e-3
    o1 = sageattention.sageattn(q, k, v, is_causal=True)
    o2 = sageattention.sageattn(q, k, 2 * v, is_causal=True)
    assert float((o2.float() - 2 * o1.float()).abs().max()) <= 4e-3
    # row 0 of a causal attention attends to key 0 only
    assert torch.allclose(o1[:, :, 0].float(), v[:, :, 0].float(), atol=1e-3)


def test_errors_are_loud():
    import sageattention
    from sageattention import _capi
    cuda_or_fail()
    q, k, v = make_qkv(1, 2, 2, 64, 64, torch.float16, "HND", seed=1)
    with pytest.raises(ValueError):
        sageattention.sageattn(q, k, v.float())
    with pytest.raises(ValueError):
        sageattention.sageattn(q, k, v, tensor_layout="XYZ")
    with pytest.raises(ValueError):
        sageattention.sageattn(q, k, v, pv_accum_dtype="fp64")
    with pytest.raises(ValueError):
        sageattention.sageattn(q, k, v[:, :, :32])
    with pytest.raises(_capi.SageB200Error):      # a grouping no kernel is built for: WARPK != BLKK
        sageattention.core._sageattn_configured(q, k, v, "HND", False, "fp32", True, False, False, (128, 64, 32, 32))


# ---------------------------------------------------------------------------------------------------
# fp8 (e4m3) P.V variant (the video-DiT case's second variant).  The reference tree has no fp8 kernel
# (parity unpinned): the checks are against the CPU emulation of the same scheme and against the
# fp16-P.V result.
# ---------------------------------------------------------------------------------------------------
def test_quant_v_fp8_matches_oracle_bit_for_bit():
    from sageattention import quant
    cuda_or_fail()
    for layout, dtype, D in (("HND", torch.bfloat16, 128), ("NHD", torch.float16, 64)):
        _, _, v = make_qkv(2, 3, 3, 777, D, dtype, layout, seed=21)
        vq, vs = quant.quant_v_fp8(v, layout)
        eq, es = O.quant_v_fp8(v.cpu(), layout)
        assert vq.dtype == torch.float8_e4m3fn and vq.shape == v.shape and vs.shape == (2, 3, D)
        assert torch.equal(vs.cpu().view(torch.int32), es.view(torch.int32))
        assert torch.equal(vq.cpu().view(torch.uint8), eq.view(torch.uint8))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D,dtype,layout,N,cfg", [(128, torch.bfloat16, "HND", 1000, CFG), (64, torch.float16, "NHD", 512, CFG),
                                                  (128, torch.float16, "HND", 2320, CFG),
                                                  (256, torch.bfloat16, "NHD", 900, CFG),
                                                  (128, torch.float16, "HND", 700, (128, 32, 32, 32))])
def test_fp8_core_matches_oracle(D, dtype, layout, N, cfg, causal):
    from sageattention import quant
    from sageattention.core import attn_fwd_quantized
    cuda_or_fail()
    q, k, v = make_qkv(1, 4, 2, N, D, dtype, layout, seed=N + D, k_bias=2.0)
    km = quant.mean_k(k, layout)
    q8, qs, k8, ks = quant.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], tensor_layout=layout, div="ieee")
    vq, vs = quant.quant_v_fp8(v, layout)
    out = torch.empty_like(q)
    lse = attn_fwd_quantized(q8, k8, vq, out, qs, ks, layout, causal, D ** -0.5, cfg, "fp32", True, "per_thread", vs)
    torch.cuda.synchronize()
    exp, exp_lse = O.attend_fp8(q8.cpu(), k8.cpu(), vq.cpu(), vs.cpu(), qs.cpu(), ks.cpu(), layout, causal,
                                BLKQ=cfg[0], WARPQ=cfg[2], BLKK=cfg[1], WARPK=cfg[3], out_dtype=dtype, return_lse=True)
    # e4m3 keeps 3 mantissa bits: where the kernel's 2^x and the emulation's differ in the last place, P
    # can round to neighbouring e4m3 values 6-12 % apart, which early causal rows (few keys) do not
    # average out - hence the wider max-abs bound for this variant; the cosine bound is unchanged
    _assert_close(out, exp, ("fp8", D, dtype, layout, N, cfg, causal), max_abs=5e-2)
    assert float((lse.cpu() - exp_lse).abs().max()) <= 2e-2


def test_fp8_api_close_to_fp16_pv_and_exact_attention():
    import sageattention
    cuda_or_fail()
    assert sageattention.sageattn_qk_int8_pv_fp8_cuda is not None
    q, k, v = make_qkv(1, 4, 4, 2320, 128, torch.bfloat16, "HND", seed=3, k_bias=2.0)
    o8, lse8 = sageattention.sageattn_qk_int8_pv_fp8_cuda(q, k, v, tensor_layout="HND", return_lse=True)
    o16, lse16 = sageattention.sageattn(q, k, v, tensor_layout="HND", return_lse=True)
    exact, _ = O.sdpa_fp32(q.cpu(), k.cpu(), v.cpu(), "HND", False)
    c = O.compare(o8.cpu(), o16.cpu())
    assert c["cos"] >= 0.999 and c["max_abs"] <= 5e-2, c
    assert O.compare(o8.cpu(), exact)["fro_rel"] <= 0.05
    assert float((lse8 - lse16).abs().max()) <= 1e-3


def test_sageattn_traces_under_torch_compile():
    """torch.compile(fullgraph=True) goes through the registered custom op and its fake implementation
    (the reference tests the same property, tests/test_sageattn_compile.py:21-31)."""
    import sageattention
    cuda_or_fail()
    q, k, v = make_qkv(1, 2, 2, 256, 64, torch.float16, "HND", seed=5)

    def fn(q, k, v):
        return sageattention.sageattn(q, k, v, tensor_layout="HND", is_causal=True) * 2.0

    compiled = torch.compile(fn, fullgraph=True, backend="aot_eager")
    got = compiled(q, k, v)
    exp = fn(q, k, v)
    assert got.shape == q.shape and torch.allclose(got.float(), exp.float(), atol=1e-3)


@pytest.mark.parametrize("mode", ["fp32", "fp16+fp32"])
def test_sageattn_per_warp_granularity(mode):
    """qk_quant_gran="per_warp": one Q scale per WARPQ = 32 rows, one K scale per BLKK = 64 keys.  The
    reference tree has no kernel of that name (parity unpinned); it is the per-block scheme with
    32-row Q blocks, so the oracle's per-block quantiser and attention with BLKQ = 32 are the check."""
    import sageattention
    cuda_or_fail()
    q, k, v = make_qkv(1, 4, 2, 1100, 128, torch.float16, "HND", seed=41, k_bias=1.0)
    out = sageattention.sageattn(q, k, v, is_causal=True, pv_accum_dtype=mode, qk_quant_gran="per_warp")
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    km = O.mean_k(kc, "HND")
    q8, qs, k8, ks = O.quant_per_block(qc, kc, km, 32, 64, "HND")
    assert qs.shape == (1, 4, -(-1100 // 32)) and ks.shape == (1, 2, -(-1100 // 64))
    exp = O.attend(q8, k8, vc, qs, ks, "HND", True, None, mode, "per_block", 32, 32, 64, 64, torch.float16)
    _assert_close(out, exp, ("per_warp", mode))
    ref, _ = O.sdpa_fp32(qc, kc, vc, "HND", True)
    c = O.compare(out.cpu(), ref)
    assert c["fro_rel"] <= 0.02 and c["max_abs"] <= 0.1, c
    # WARPQ = 16 (the reference's (128, 64, 16, 64) candidate): one Q scale per 16 rows
    from sageattention.core import _sageattn_configured
    out16 = _sageattn_configured(q, k, v, "HND", True, mode, True, False, False, (128, 64, 16, 64), None, "per_warp")
    q8, qs, k8, ks = O.quant_per_block(qc, kc, km, 16, 64, "HND")
    exp16 = O.attend(q8, k8, vc, qs, ks, "HND", True, None, mode, "per_block", 16, 16, 64, 64, torch.float16)
    _assert_close(out16, exp16, ("per_warp 16", mode))


@pytest.mark.parametrize("mode", ["fp32", "fp16+fp32", "fp16"])
def test_results_are_reproducible_bit_for_bit(mode):
    """The same call gives the same bits every time, although the softmax warpgroups of a CTA run
    unsynchronised (which CTA runs where, and how the warpgroups interleave, changes from run to run)."""
    import sageattention
    cuda_or_fail()
    q, k, v = make_qkv(1, 8, 4, 4096, 128, torch.float16, "HND", seed=51, k_bias=1.0)
    outs = [sageattention.sageattn(q, k, v, is_causal=True, pv_accum_dtype=mode) for _ in range(5)]
    torch.cuda.synchronize()
    assert all(torch.equal(outs[0], o) for o in outs[1:])


def test_sageattn_can_be_captured_in_a_cuda_graph(monkeypatch):
    """The whole call (quantisers, K mean, attention) allocates through torch's caching allocator and
    enqueues on the current stream only, so it can be captured once and replayed: the replay on new
    inputs written into the captured buffers gives exactly the eager result."""
    import sageattention
    cuda_or_fail()
    monkeypatch.setenv("SAGE_B200_CHECK", "0")          # reading the status word back would synchronise
    q, k, v = make_qkv(1, 4, 2, 1536, 128, torch.bfloat16, "NHD", seed=31, k_bias=1.0)
    kw = dict(tensor_layout="NHD", is_causal=True, pv_accum_dtype="fp16+fp32")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):                               # warm-up outside the capture (function attributes, allocator)
            sageattention.sageattn(q, k, v, **kw)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_g = sageattention.sageattn(q, k, v, **kw)
    q2, k2, v2 = make_qkv(1, 4, 2, 1536, 128, torch.bfloat16, "NHD", seed=32, k_bias=1.0)
    q.copy_(q2), k.copy_(k2), v.copy_(v2)
    graph.replay()
    torch.cuda.synchronize()
    eager = sageattention.sageattn(q2, k2, v2, **kw)
    assert torch.equal(out_g, eager)


def test_random_shapes_agree_across_accumulate_modes():
    """150 seeded random problems (batch, GQA ratio, lengths from 1 to 6000 with unequal query/key
    lengths, head_dim incl. padded ones and 256, both layouts and dtypes, causal or not, LSE or not):
    every mode finishes with a clean status word, finite output, and agrees with the fp32 mode."""
    import random
    import sageattention
    cuda_or_fail()
    rng = random.Random(1234)
    for _ in range(150):
        B = rng.choice([1, 1, 2, 3])
        Hkv = rng.choice([1, 2, 4, 8])
        Hq = Hkv * rng.choice([1, 1, 2, 4])
        D = rng.choice([64, 128, 128, 128, 256, 96, 40])
        N = rng.choice([1, 7, 64, 127, 128, 129, 255, 256, 300, 511, 777, 1024, 1500, 2049, 4096, 6000])
        Nkv = N if rng.random() < 0.8 else rng.choice([64, 200, 1000, 3000])
        dtype = rng.choice([torch.float16, torch.bfloat16])
        layout = rng.choice(["HND", "NHD"])
        causal = rng.random() < 0.5
        mode = rng.choice(["fp16+fp32", "fp16+fp32", "fp16"])
        gen = torch.Generator(device="cuda").manual_seed(rng.randrange(1 << 30))      # on the device: this test is about shapes
        shp = (lambda h, n: (B, h, n, D)) if layout == "HND" else (lambda h, n: (B, n, h, D))
        q = torch.randn(shp(Hq, N), device="cuda", generator=gen).to(dtype)
        k = (torch.randn(shp(Hkv, Nkv), device="cuda", generator=gen) + rng.choice([0.0, 2.0])).to(dtype)
        v = torch.randn(shp(Hkv, Nkv), device="cuda", generator=gen).to(dtype)
        out = sageattention.sageattn(q, k, v, tensor_layout=layout, is_causal=causal, pv_accum_dtype=mode,
                                     return_lse=rng.random() < 0.3)
        out = out[0] if isinstance(out, tuple) else out
        ref = sageattention.sageattn(q, k, v, tensor_layout=layout, is_causal=causal, pv_accum_dtype="fp32")
        what = (B, Hq, Hkv, N, Nkv, D, dtype, layout, causal, mode)
        assert bool(torch.isfinite(out.float()).all()), what
        c = O.compare(out.float().cpu(), ref.float().cpu())
        assert c["cos"] > 0.9995, (what, c)


@pytest.mark.parametrize("mode", ["fp32", "fp16+fp32", "fp16"])
def test_extreme_score_ranges(mode):
    """Scores spread over hundreds of binades (large inputs, sm_scale = 1): the running maximum jumps by
    far more than fp16 or the rescale factors can represent between blocks, rows become one-hot, and
    factors underflow to zero.  Output and LSE must still follow the oracle."""
    cuda_or_fail()
    q, k, v = make_qkv(1, 2, 2, 1024, 128, torch.float16, "HND", seed=61)
    q, k = q * 4.0, k * 4.0
    out, lse, qz = _run_core(q, k, v, "HND", True, mode, sm_scale=1.0, return_lse=True)
    exp, exp_lse = _oracle(qz, "HND", True, mode, "per_thread", torch.float16, sm_scale=1.0)
    assert bool(torch.isfinite(out.float()).all()) and bool(torch.isfinite(lse).all())
    _assert_close(out, exp, ("extreme", mode))
    assert float(((lse.cpu() - exp_lse).abs() / exp_lse.abs().clamp_min(1.0)).max()) <= 1e-3



@pytest.mark.parametrize("layout,Hq,Hkv,chunk", [("HND", 12, 6, None), ("HND", 10, 5, 2), ("NHD", 8, 4, 3)])
def test_host_buffer_entry_point_equals_the_device_call(layout, Hq, Hkv, chunk):
    """sageattn_host (host tensors in, host tensor out, pipelined over groups of kv-heads) returns the
    bits of one sageattn call on the whole tensors: heads are independent and the kernels are
    deterministic, whatever the grouping (default, ragged last group, non-contiguous NHD slices).
    (At this length the K mean adds its rows in the same order for any head count; for long sequences
    the row split follows the number of heads in the call and the mean may move by one rounding.)"""
    import sageattention
    from sageattention.host import sageattn_host
    cuda_or_fail()
    q, k, v = make_qkv(2, Hq, Hkv, 1000, 128, torch.float16, layout, seed=77, k_bias=1.0, device="cpu")
    q, k, v = q.pin_memory(), k.pin_memory(), v.pin_memory()
    got = sageattn_host(q, k, v, tensor_layout=layout, kv_heads_per_chunk=chunk, is_causal=True)
    exp = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), tensor_layout=layout, is_causal=True)
    torch.cuda.synchronize()
    assert not got.is_cuda and got.shape == q.shape and got.dtype == q.dtype
    assert torch.equal(got, exp.cpu())
    with pytest.raises(ValueError):
        sageattn_host(q.cuda(), k, v)


def test_host_buffer_entry_point_replays_a_captured_step():
    """With pinned buffers whose head groups are contiguous the second call with the same tensors replays a
    CUDA graph of the whole pipelined step: same bits as the step-by-step call, and new contents of the
    same buffers are picked up."""
    import sageattention
    from sageattention import host
    cuda_or_fail()
    q, k, v = make_qkv(1, 12, 6, 1000, 128, torch.float16, "HND", seed=78, k_bias=1.0, device="cpu")
    q, k, v = q.pin_memory(), k.pin_memory(), v.pin_memory()
    out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    kw = dict(tensor_layout="HND", kv_heads_per_chunk=2, is_causal=True)
    first = host.sageattn_host(q, k, v, out=out, **kw).clone()
    plan = next(reversed(host._plans.values()))
    assert plan.graph is not None, "the step was not captured"
    second = host.sageattn_host(q, k, v, out=out, **kw).clone()
    exp = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), tensor_layout="HND", is_causal=True).cpu()
    assert torch.equal(first, exp) and torch.equal(second, exp)
    q.neg_()                                                   # same buffers, new contents
    third = host.sageattn_host(q, k, v, out=out, **kw)
    exp3 = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), tensor_layout="HND", is_causal=True).cpu()
    assert torch.equal(third, exp3) and not torch.equal(exp3, exp)
