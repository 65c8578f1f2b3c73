"""GPU parity at the full benchmark shapes, compared on the device.

The same int8 tensors and scales go into the reference's sm80 CUDA kernel (its sources compiled for
sm_100 under oracle/_ref) and into this library's kernel; outputs are compared with torch on the GPU
(cosine >= 0.9995, max-abs <= 2e-2; for bf16 outputs one bf16 ulp where that is larger).  The
quantisers are compared bit for bit with the reference's Triton kernels (compiled to sm_100a cubins
under oracle/_ref/triton_quant) on the same inputs and the same K mean.

Shapes:
  SD      B=16 H=10  N=4096  D=64  fp16 HND, K offset N(0, 3^2), non-causal
  GQA     B=4  Hq=32 Hkv=8 N=8192 D=128 bf16 NHD, 4 outlier channels x20, causal, LSE
  DiT     B=1  H=24 (a few heads for attention) N=75600 D=128 bf16 HND, K bias N(0, 2^2), non-causal
  LONG    B=1  H=64  N=32768 (and 65536 with a few heads) D=128 fp16 HND, causal
Inputs are seeded and generated on the device.
"""
import pytest
import torch

from gpu_util import cuda_or_fail, reference_ops

pytestmark = pytest.mark.gpu

COS_MIN = 0.9995
MAX_ABS = 2e-2
CFG = (128, 64, 32, 64)
REF_OP = {"fp32": "qk_int8_sv_f16_accum_f32_attn", "fp16+fp32": "qk_int8_sv_f16_accum_f16_attn_inst_buf",
          "fp16": "qk_int8_sv_f16_accum_f16_attn"}


def device_qkv(B, Hq, Hkv, N, D, dtype, layout, seed, k_bias=0.0, k_outliers=0.0):
    dev = cuda_or_fail()
    g = torch.Generator(device=dev).manual_seed(seed)

    def shape(h):
        return (B, h, N, D) if layout == "HND" else (B, N, h, D)
    q = torch.randn(shape(Hq), generator=g, device=dev).to(dtype)
    k = torch.randn(shape(Hkv), generator=g, device=dev)
    v = torch.randn(shape(Hkv), generator=g, device=dev).to(dtype)
    if k_bias:
        k += k_bias * torch.randn((1, Hkv, 1, D) if layout == "HND" else (1, 1, Hkv, D), generator=g, device=dev)
    if k_outliers:
        for h in range(Hkv):
            ch = torch.randperm(D, generator=g, device=dev)[:4]
            if layout == "HND":
                k[:, h, :, ch] *= k_outliers
            else:
                k[:, :, h, ch] *= k_outliers
    return q, k.to(dtype), v


def close_on_device(got, exp, what, max_abs=MAX_ABS, cos_min=COS_MIN):
    """The tolerance of the parity tests, evaluated on the GPU (the tensors are too large to bring back)."""
    g, e = got.float().flatten(), exp.float().flatten()
    cos = float(torch.dot(g, e) / (g.norm() * e.norm()).clamp_min(1e-30))
    bound = torch.full_like(e, max_abs)
    if exp.dtype == torch.bfloat16:
        ulp = torch.exp2(torch.floor(torch.log2(e.abs().clamp_min(1e-30))) - 7)
        bound = torch.maximum(bound, ulp)
    diff = (g - e).abs()
    worst = float((diff - bound).max())
    assert bool(torch.isfinite(g).all()), what
    assert cos >= cos_min and worst <= 0.0, (what, cos, float(diff.max()))
    return cos, float(diff.max())


def quantise(q, k, v, layout, cfg=CFG):
    from sageattention import quant
    km = k.mean(dim=2 if layout == "HND" else 1, keepdim=True)       # the reference's own expression
    q8, qs, k8, ks = quant.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], layout, div="full")
    return q8, qs, k8, ks, quant.cast_v_fp16(v, layout), km


def ours_and_reference(qz, like, layout, causal, mode, cfg=CFG, return_lse=False):
    from sageattention.core import attn_fwd_quantized
    ref = reference_ops()
    assert ref is not None, "oracle/_ref/libsage_ref_sm80.so is missing: run make -C oracle"
    q8, qs, k8, ks, v16 = qz
    out = torch.empty_like(like)
    lse = attn_fwd_quantized(q8, k8, v16, out, qs, ks, layout, causal, like.size(-1) ** -0.5, cfg, mode, return_lse)
    ref_out = torch.empty_like(like)
    getattr(ref, REF_OP[mode])(q8, k8, v16, ref_out, qs, ks, 0 if layout == "NHD" else 1, causal,
                               like.size(-1) ** -0.5, *cfg, False)
    torch.cuda.synchronize()
    return out, ref_out, lse


def dequantised_scores_lse(q8, qs, k8, ks, b, h, h_kv, layout, causal, sm_scale, cfg=CFG):
    """log2-sum-exp2 of one head's scores rebuilt from the int8 tensors and per-thread scales in fp32
    on the device: the quantity the kernel's LSE output is defined as."""
    blk_q, blk_k, warp_q, warp_k = cfg
    qh = (q8[b, h] if layout == "HND" else q8[b, :, h]).float()
    kh = (k8[b, h_kv] if layout == "HND" else k8[b, :, h_kv]).float()
    nq, nk = qh.size(0), kh.size(0)
    r = torch.arange(nq, device=qh.device)
    c = torch.arange(nk, device=qh.device)
    q_sc = qs[b, h][(r // warp_q) * 8 + (r % 8)]
    k_sc = ks[b, h_kv][(c // warp_k) * 4 + (c % 8) // 2]
    s = (qh @ kh.t()) * q_sc[:, None] * k_sc[None, :] * (sm_scale * 1.4426950408889634)
    if causal:
        s = s.masked_fill(c[None, :] > r[:, None], float("-inf"))
    m = s.amax(dim=1, keepdim=True)
    return (torch.log2(torch.exp2(s - m).sum(dim=1)) + m.squeeze(1))


# ----------------------------------------------------------------------------------------- attention
@pytest.mark.parametrize("mode", ["fp16+fp32", "fp32", "fp16"])
def test_sd_shape_matches_reference_kernel(mode):
    q, k, v = device_qkv(16, 10, 10, 4096, 64, torch.float16, "HND", seed=1, k_bias=3.0)
    q8, qs, k8, ks, v16, _ = quantise(q, k, v, "HND")
    out, ref_out, _ = ours_and_reference((q8, qs, k8, ks, v16), q, "HND", False, mode)
    print("sd", mode, close_on_device(out, ref_out, ("sd", mode)))


@pytest.mark.parametrize("B,H,N,D,causal,dtype", [(1, 16, 6000, 128, True, torch.float16),       # persistent one-tile kernel
                                                  (1, 16, 6200, 128, True, torch.bfloat16),      # one CTA per tile
                                                  (2, 10, 8100, 64, False, torch.float16),       # persistent at 64 channels
                                                  (1, 8, 8300, 128, False, torch.float16),       # one CTA per tile, no mask
                                                  (1, 10, 16500, 64, False, torch.bfloat16)])
def test_lengths_around_the_tables_kernel_switch_match_reference_kernel(B, H, N, D, causal, dtype):
    """Key lengths on both sides of the tile table's switch between the persistent one-tile kernel and one
    CTA per tile (causal: 6144 keys at 128 channels, 8192 at 64; otherwise 8192 and 16384), ragged on purpose."""
    from sageattention.tile_table import select_entry
    q, k, v = device_qkv(B, H, H, N, D, dtype, "HND", seed=11, k_bias=1.0)
    q8, qs, k8, ks, v16, _ = quantise(q, k, v, "HND")
    out, ref_out, lse = ours_and_reference((q8, qs, k8, ks, v16), q, "HND", causal, "fp16+fp32", return_lse=True)
    kernel = select_entry(D, causal, "fp16+fp32", N)["kernel"]
    print(N, D, kernel, close_on_device(out, ref_out, (N, D, kernel)))
    exp = dequantised_scores_lse(q8, qs, k8, ks, B - 1, H - 1, H - 1, "HND", causal, D ** -0.5)
    assert float((lse[B - 1, H - 1] - exp).abs().max()) <= 2e-2


def test_gqa_prefill_shape_matches_reference_kernel_and_lse():
    q, k, v = device_qkv(4, 32, 8, 8192, 128, torch.bfloat16, "NHD", seed=2, k_outliers=20.0)
    q8, qs, k8, ks, v16, _ = quantise(q, k, v, "NHD")
    out, ref_out, lse = ours_and_reference((q8, qs, k8, ks, v16), q, "NHD", True, "fp32", return_lse=True)
    print("gqa", close_on_device(out, ref_out, "gqa fp32"))
    assert lse.shape == (4, 32, 8192)
    for b, h in ((0, 0), (3, 31), (1, 13)):
        exp = dequantised_scores_lse(q8, qs, k8, ks, b, h, h // 4, "NHD", True, 128 ** -0.5)
        assert float((lse[b, h] - exp).abs().max()) <= 2e-2, (b, h)


@pytest.mark.parametrize("mode", ["fp32", "fp16+fp32", "fp16"])
def test_dit_length_matches_reference_kernel(mode):
    """N = 75600 is not a multiple of any tile: 590 full key blocks and a tail of 80 keys, a last query
    tile of 80 rows."""
    q, k, v = device_qkv(1, 3, 3, 75600, 128, torch.bfloat16, "HND", seed=3, k_bias=2.0)
    q8, qs, k8, ks, v16, _ = quantise(q, k, v, "HND")
    out, ref_out, _ = ours_and_reference((q8, qs, k8, ks, v16), q, "HND", False, mode)
    print("dit", mode, close_on_device(out, ref_out, ("dit", mode)))


def test_dit_length_fp8_pv_close_to_fp16_pv():
    """The e4m3 P.V variant at N = 75600 against the fp16 P.V result of the same call (the reference
    tree has no fp8 kernel to compare with)."""
    import sageattention
    q, k, v = device_qkv(1, 3, 3, 75600, 128, torch.bfloat16, "HND", seed=3, k_bias=2.0)
    o8 = sageattention.sageattn_qk_int8_pv_fp8_cuda(q, k, v, tensor_layout="HND")
    o16 = sageattention.sageattn(q, k, v, tensor_layout="HND", pv_accum_dtype="fp32")
    torch.cuda.synchronize()
    print("dit fp8", close_on_device(o8, o16, "dit fp8 vs fp16 pv", max_abs=5e-2, cos_min=0.999))


@pytest.mark.parametrize("mode", ["fp16+fp32", "fp32"])
def test_long_context_all_heads_match_reference_kernel(mode):
    """The headline shape: 64 heads, N = 32768, causal."""
    q, k, v = device_qkv(1, 64, 64, 32768, 128, torch.float16, "HND", seed=4)
    q8, qs, k8, ks, v16, _ = quantise(q, k, v, "HND")
    del k
    out, ref_out, _ = ours_and_reference((q8, qs, k8, ks, v16), q, "HND", True, mode)
    print("long 32k", mode, close_on_device(out, ref_out, ("long 32k", mode)))


def test_long_context_64k_matches_reference_kernel():
    q, k, v = device_qkv(1, 4, 4, 65536, 128, torch.float16, "HND", seed=5)
    q8, qs, k8, ks, v16, _ = quantise(q, k, v, "HND")
    out, ref_out, lse = ours_and_reference((q8, qs, k8, ks, v16), q, "HND", True, "fp16+fp32", return_lse=True)
    print("long 64k", close_on_device(out, ref_out, "long 64k"))
    exp = dequantised_scores_lse(q8[:, :, :16384], qs, k8[:, :, :16384], ks, 0, 2, 2, "HND", True, 128 ** -0.5)
    assert float((lse[0, 2, :16384] - exp).abs().max()) <= 2e-2


@pytest.mark.parametrize("cfg", [(64, 64, 32, 64), (128, 64, 16, 64)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("mode", ["fp32", "fp16+fp32", "fp16"])
def test_other_per_thread_groupings_match_reference_kernel(cfg, causal, mode):
    """The reference's (BLKQ, BLKK, WARPQ, WARPK) candidates with 64-row query blocks and with 16-row
    warps (sageattention/cuda_autotune.py:11-13): Q scales per 8 x 4 and per 8 x 2 rows."""
    for D, dtype, layout, N in ((128, torch.float16, "HND", 4096), (64, torch.bfloat16, "NHD", 2320)):
        q, k, v = device_qkv(2, 4, 2, N, D, dtype, layout, seed=N + cfg[0] + cfg[2], k_bias=1.0)
        q8, qs, k8, ks, v16, _ = quantise(q, k, v, layout, cfg)
        out, ref_out, _ = ours_and_reference((q8, qs, k8, ks, v16), q, layout, causal, mode, cfg)
        close_on_device(out, ref_out, (cfg, causal, mode, D))


# ----------------------------------------------------------------------------------------- quantisers
QUANT_SHAPES = {
    "sd": dict(B=16, Hq=10, Hkv=10, N=4096, D=64, dtype=torch.float16, layout="HND", seed=1, k_bias=3.0),
    "gqa": dict(B=4, Hq=32, Hkv=8, N=8192, D=128, dtype=torch.bfloat16, layout="NHD", seed=2, k_outliers=20.0),
    "dit": dict(B=1, Hq=24, Hkv=24, N=75600, D=128, dtype=torch.bfloat16, layout="HND", seed=3, k_bias=2.0),
    "long": dict(B=1, Hq=64, Hkv=64, N=32768, D=128, dtype=torch.float16, layout="HND", seed=4),
}


@pytest.mark.parametrize("name", sorted(QUANT_SHAPES))
def test_quantisers_bit_exact_with_reference_triton_kernels_at_full_size(name):
    """Every grouping the reference can select, at the full benchmark shapes: int8 values and scales equal
    those of the reference's own kernels on this GPU, bit for bit.  N = 75600 ends in a 16-row tail
    whose masked rows still take part in the maximum through the subtracted mean."""
    from oracle import triton_ref
    from sageattention import quant
    assert triton_ref.available(), "oracle/_ref/triton_quant is missing: run python oracle/build_triton_ref.py"
    a = QUANT_SHAPES[name]
    q, k, _ = device_qkv(**a)
    layout = a["layout"]
    km = k.mean(dim=2 if layout == "HND" else 1, keepdim=True)
    for cfg in [(128, 64, 32, 64), (128, 32, 32, 32), (64, 64, 32, 64), (128, 64, 16, 64)]:
        exp = triton_ref.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], layout)
        got = quant.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], layout, div="full")
        torch.cuda.synchronize()
        for i, what in enumerate(("q_int8", "q_scale", "k_int8", "k_scale")):
            a_, b_ = (got[i], exp[i]) if i % 2 == 0 else (got[i].view(torch.int32), exp[i].view(torch.int32))
            assert torch.equal(a_, b_), (name, cfg, what, int((a_ != b_).sum()))
        del exp, got
    exp = triton_ref.per_block_int8(q, k, km, 128, 64, layout)
    got = quant.per_block_int8(q, k, km, 128, 64, layout, div="full")
    torch.cuda.synchronize()
    for i, what in enumerate(("q_int8", "q_scale", "k_int8", "k_scale")):
        a_, b_ = (got[i], exp[i]) if i % 2 == 0 else (got[i].view(torch.int32), exp[i].view(torch.int32))
        assert torch.equal(a_, b_), (name, "per_block", what, int((a_ != b_).sum()))
