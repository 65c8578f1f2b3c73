"""GPU parity of the quantisation front end (through the C ABI) - bit-exact gates.

1. against the golden vectors produced by the reference's Triton kernels (IEEE division mode);
2. against the CPU oracle on seeded inputs with ragged and tiny lengths (IEEE mode);
3. against the reference's Triton kernels compiled for sm_100a and run on the same GPU
   (div.full mode) when oracle/_ref/triton_quant is present.
"""
import numpy as np
import pytest
import torch

import golden_io as G
from gpu_util import cuda_or_fail, make_qkv
from oracle import sage_oracle as O

pytestmark = pytest.mark.gpu


def _eq(a, b):
    return torch.equal(a.cpu(), b.cpu() if isinstance(b, torch.Tensor) else torch.from_numpy(b))


def _eq_bits(a, b):
    b = b if isinstance(b, torch.Tensor) else torch.from_numpy(b)
    return torch.equal(a.cpu().view(torch.int32), b.cpu().view(torch.int32))


@pytest.mark.parametrize("name", G.names())
def test_quant_matches_golden_vectors(name):
    from sageattention import quant
    dev = cuda_or_fail()
    g = G.load(name)
    r = g["raw"]
    q, k = g["q"].to(dev), g["k"].to(dev)
    km = g["km"].to(dev) if g["km"] is not None else None
    for cfg in G.PER_THREAD_CONFIGS:
        tag = "pt_%d_%d_%d_%d" % cfg
        q8, qs, k8, ks = quant.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], g["layout"], div="ieee")
        assert qs.shape == r[tag + "_qs"].shape and ks.shape == r[tag + "_ks"].shape
        assert _eq_bits(qs, r[tag + "_qs"]), (name, tag, "q_scale")
        assert _eq_bits(ks, r[tag + "_ks"]), (name, tag, "k_scale")
        if tag + "_q8" in r:
            assert _eq(q8, r[tag + "_q8"]) and _eq(k8, r[tag + "_k8"]), (name, tag)
        assert [int(q8.long().sum()), int((q8.long() ** 2).sum())] == list(r[tag + "_q8sum"])
        assert [int(k8.long().sum()), int((k8.long() ** 2).sum())] == list(r[tag + "_k8sum"])
    q8, qs, k8, ks = quant.per_block_int8(q, k, km, 128, 64, g["layout"], div="ieee")
    assert _eq_bits(qs, r["pb_128_64_qs"]) and _eq_bits(ks, r["pb_128_64_ks"])
    assert _eq(q8, r["pb_128_64_q8"]) and _eq(k8, r["pb_128_64_k8"])


@pytest.mark.parametrize("N", [1, 7, 63, 64, 65, 127, 128, 129, 200, 1000])
@pytest.mark.parametrize("D,dtype,layout", [(64, torch.float16, "HND"), (128, torch.bfloat16, "NHD"),
                                             (256, torch.float16, "NHD")])
def test_quant_matches_oracle_on_ragged_lengths(N, D, dtype, layout):
    from sageattention import quant
    cuda_or_fail()
    q, k, _ = make_qkv(2, 4, 2, N, D, dtype, layout, seed=100 + N, k_bias=1.5)
    km = quant.mean_k(k, layout)
    qc, kc, kmc = q.cpu(), k.cpu(), km.cpu()
    for cfg in [(128, 64, 32, 64), (64, 64, 32, 64), (128, 64, 16, 64), (128, 32, 32, 32)]:
        got = quant.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], layout, div="ieee")
        exp = O.quant_per_thread(qc, kc, kmc, cfg[0], cfg[2], cfg[1], cfg[3], layout)
        assert _eq(got[0], exp[0]) and _eq_bits(got[1], exp[1]), (cfg, "q")
        assert _eq(got[2], exp[2]) and _eq_bits(got[3], exp[3]), (cfg, "k")
    got = quant.per_block_int8(q, k, km, 128, 64, layout, div="ieee")
    exp = O.quant_per_block(qc, kc, kmc, 128, 64, layout)
    assert _eq(got[0], exp[0]) and _eq_bits(got[1], exp[1])
    assert _eq(got[2], exp[2]) and _eq_bits(got[3], exp[3])
    # no smoothing
    got = quant.per_thread_int8(q, k, None, tensor_layout=layout, div="ieee")
    exp = O.quant_per_thread(qc, kc, None, tensor_layout=layout)
    assert _eq(got[2], exp[2]) and _eq_bits(got[3], exp[3])


@pytest.mark.parametrize("D,dtype,layout,N", [(128, torch.bfloat16, "NHD", 1000), (64, torch.float16, "HND", 777),
                                              (128, torch.float16, "HND", 4096)])
def test_quant_matches_reference_triton_kernels_on_gpu(D, dtype, layout, N):
    """div.full mode against the reference's own kernels compiled for sm_100a."""
    from oracle import triton_ref
    from sageattention import quant
    cuda_or_fail()
    assert triton_ref.available(), "oracle/_ref/triton_quant is missing: run python oracle/build_triton_ref.py"
    q, k, _ = make_qkv(2, 4, 2, N, D, dtype, layout, seed=N, k_bias=2.0, k_outliers=20.0)
    km = k.mean(dim=2 if layout == "HND" else 1, keepdim=True)
    for cfg in [(128, 64, 32, 64), (128, 64, 16, 64), (128, 32, 32, 32)]:
        exp = triton_ref.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], layout)
        got = quant.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], layout, div="full")
        torch.cuda.synchronize()
        for i, what in enumerate(("q_int8", "q_scale", "k_int8", "k_scale")):
            same = _eq(got[i], exp[i]) if i % 2 == 0 else _eq_bits(got[i], exp[i])
            assert same, (cfg, what, int((got[i] != exp[i]).sum()))
    exp = triton_ref.per_block_int8(q, k, km, 128, 64, layout)
    got = quant.per_block_int8(q, k, km, 128, 64, layout, div="full")
    for i, what in enumerate(("q_int8", "q_scale", "k_int8", "k_scale")):
        same = _eq(got[i], exp[i]) if i % 2 == 0 else _eq_bits(got[i], exp[i])
        assert same, ("per_block", what, int((got[i] != exp[i]).sum()))


@pytest.mark.parametrize("D,dtype,layout,N", [(128, torch.bfloat16, "HND", 75600), (64, torch.float16, "NHD", 4096),
                                              (128, torch.float16, "NHD", 333)])
def test_mean_k_within_one_ulp_of_torch(D, dtype, layout, N):
    from sageattention import quant
    cuda_or_fail()
    _, k, _ = make_qkv(1, 1, 3, N, D, dtype, layout, seed=N, k_bias=2.0)
    km = quant.mean_k(k, layout)
    ref64 = k.double().mean(dim=2 if layout == "HND" else 1, keepdim=True)
    ref = ref64.to(dtype)
    assert km.shape == ref.shape and km.dtype == dtype
    # distance in units of the 16-bit type's spacing at the value
    a = km.view(torch.int16).int()
    b = ref.view(torch.int16).int()
    assert int((a - b).abs().max()) <= 1
    assert float((a != b).float().mean()) < 0.05


@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_mean_k_does_not_depend_on_the_grouping_of_heads(layout):
    """A (batch, head) plane's mean has the same bits whether it is reduced with the whole tensor or
    alone (a head group of the pipelined host call, a rank's shard of the heads): the row split
    follows the sequence length only.  Long enough for many splits per plane."""
    from sageattention import quant
    cuda_or_fail()
    _, k, _ = make_qkv(2, 6, 6, 20000, 128, torch.bfloat16, layout, seed=17, k_bias=2.0)
    full = quant.mean_k(k, layout)
    hdim = 1 if layout == "HND" else 2
    for lo, hi in ((0, 1), (1, 4), (4, 6)):
        part = quant.mean_k(k.narrow(hdim, lo, hi - lo), layout)
        assert torch.equal(part, full.narrow(hdim, lo, hi - lo)), (layout, lo, hi)
    one = quant.mean_k(k[1:2].narrow(hdim, 5, 1), layout)
    assert torch.equal(one, full[1:2].narrow(hdim, 5, 1))


def test_cast_v_is_exactly_torch_cast():
    from sageattention import quant
    cuda_or_fail()
    for layout in ("HND", "NHD"):
        _, _, v = make_qkv(2, 2, 2, 300, 128, torch.bfloat16, layout, seed=5)
        v[0, 0, 0, 0] = 70000.0     # overflows fp16
        v[0, 0, 0, 1] = 1e-7        # below fp16 normal range
        assert torch.equal(quant.cast_v_fp16(v, layout), v.to(torch.float16))
    v16 = torch.randn(1, 2, 64, 64, device="cuda").half()
    assert quant.cast_v_fp16(v16, "HND") is v16


def test_quant_idempotent_properties_at_full_size():
    """Size-independent properties at a full-length tensor: dequantised values stay within half
    a step of the input and the scale equals max|x| / 127 (+1e-7) of its group."""
    from sageattention import quant
    cuda_or_fail()
    q, k, _ = make_qkv(1, 4, 4, 32768, 128, torch.float16, "HND", seed=4)
    q8, qs, k8, ks = quant.per_thread_int8(q, k, None, div="ieee")
    B, H, N, D = q.shape
    sc = qs.view(B, H, N // 32, 1, 8, 1).expand(B, H, N // 32, 4, 8, 1).reshape(B, H, N, 1)
    err = (q8.float() * sc - q.float()).abs()
    assert bool((err <= 0.5 * sc * 1.0001 + 1e-6).all())
    # evaluated on the CPU: torch's CUDA division by a scalar multiplies by the reciprocal
    amax = q.float().abs().view(B, H, N // 32, 4, 8, D).amax(dim=(3, 5)).cpu()
    assert torch.equal(qs.view(B, H, N // 32, 8).cpu(), amax / 127.0 + 1e-7)
    assert int(q8.abs().max()) == 127


@pytest.mark.parametrize("B,H,N,layout", [(1, 6, 700, "HND"), (1, 5, 700, "NHD"), (3, 2, 700, "HND"), (3, 2, 700, "NHD"),
                                          (1, 40, 4096, "HND"), (5, 8, 4096, "NHD")])
def test_smooth_quant_k_slicing_does_not_change_results(B, H, N, layout, monkeypatch):
    """K mean + quantisation processed in L2-sized slices (of heads, or of batches) gives exactly the
    mean and the int8 values / scales of the unsliced two-step path."""
    from sageattention import _capi as C
    from sageattention import quant
    cuda_or_fail()
    # (the long cases have enough planes that a slice on its own would split its rows differently
    # from the whole tensor: the row split must follow the whole tensor)
    _, k, _ = make_qkv(B, H, H, N, 128, torch.bfloat16, layout, seed=B * 10 + H, k_bias=2.0)
    km_ref = quant.mean_k(k, layout)
    k8_ref, ks_ref = quant._quant_one(k, km_ref, 64, 64, C.GROUP_K_THREAD, layout, "full")
    for slice_bytes in (0, 1, 2 * N * 128 * 2, 8 * N * 128 * 2, 64 << 20):
        monkeypatch.setattr(quant, "_L2_SLICE_BYTES", slice_bytes)
        km, k8, ks = quant.smooth_quant_k(k, 64, 64, C.GROUP_K_THREAD, layout, "full")
        torch.cuda.synchronize()
        assert torch.equal(km, km_ref) and torch.equal(k8, k8_ref) and torch.equal(ks, ks_ref), slice_bytes
