"""CPU checks: the oracle against the reference's golden vectors, host-side logic, and the C-ABI
library's exported symbols (no compute calls - there is no GPU here)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import golden_io as G
from oracle import sage_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _same_bits(a: torch.Tensor, b: np.ndarray) -> bool:
    return np.array_equal(a.numpy().view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("name", G.names())
def test_oracle_quantisers_match_reference_bit_for_bit(name):
    g = G.load(name)
    r = g["raw"]
    for cfg in G.PER_THREAD_CONFIGS:
        tag = "pt_%d_%d_%d_%d" % cfg
        q8, qs, k8, ks = O.quant_per_thread(g["q"], g["k"], g["km"], cfg[0], cfg[2], cfg[1], cfg[3], g["layout"])
        assert _same_bits(qs, r[tag + "_qs"]) and _same_bits(ks, r[tag + "_ks"])
        assert qs.shape == r[tag + "_qs"].shape and ks.shape == r[tag + "_ks"].shape
        if tag + "_q8" in r:
            assert np.array_equal(q8.numpy(), r[tag + "_q8"]) and np.array_equal(k8.numpy(), r[tag + "_k8"])
        assert [int(q8.long().sum()), int((q8.long() ** 2).sum())] == list(r[tag + "_q8sum"])
        assert [int(k8.long().sum()), int((k8.long() ** 2).sum())] == list(r[tag + "_k8sum"])
    q8, qs, k8, ks = O.quant_per_block(g["q"], g["k"], g["km"], 128, 64, g["layout"])
    assert _same_bits(qs, r["pb_128_64_qs"]) and _same_bits(ks, r["pb_128_64_ks"])
    assert np.array_equal(q8.numpy(), r["pb_128_64_q8"]) and np.array_equal(k8.numpy(), r["pb_128_64_k8"])


@pytest.mark.parametrize("name", G.names())
def test_oracle_mean_matches_torch_mean_of_fixture(name):
    g = G.load(name)
    if g["km"] is None:
        pytest.skip("fixture without smoothing")
    assert torch.equal(O.mean_k(g["k"], g["layout"]), g["km"])


@pytest.mark.parametrize("name", [n for n in G.names() if "tri_o_bits" in G.load(n)["raw"]])
@pytest.mark.parametrize("causal", [False, True])
def test_oracle_attention_matches_reference_triton_kernel(name, causal):
    g = G.load(name)
    r = g["raw"]
    sfx = "_causal" if causal else ""
    q8 = torch.from_numpy(r["pb_128_64_q8"])
    k8 = torch.from_numpy(r["pb_128_64_k8"])
    qs = torch.from_numpy(r["pb_128_64_qs"])
    ks = torch.from_numpy(r["pb_128_64_ks"])
    o, lse = O.attend(q8, k8, g["v"].half(), qs, ks, g["layout"], causal, None, "fp32", "per_block",
                      128, 32, 64, 64, g["dtype"], True)
    ref = G.from_bits(r["tri_o_bits" + sfx], g["dtype"])
    c = O.compare(o, ref)
    assert c["cos"] >= 0.99999 and c["max_abs"] <= 2e-3, c
    assert float((lse - torch.from_numpy(r["tri_lse" + sfx])).abs().max()) <= 1e-3


def test_oracle_end_to_end_close_to_fp32_attention():
    g = torch.Generator().manual_seed(7)
    q = torch.randn(1, 2, 300, 64, generator=g).half()
    k = (torch.randn(1, 2, 300, 64, generator=g) + 2.0).half()
    v = torch.randn(1, 2, 300, 64, generator=g).half()
    for causal in (False, True):
        for mode in ("fp32", "fp16+fp32", "fp16"):
            o, lse = O.sageattn(q, k, v, "HND", causal, mode, True, True)
            ref, ref_lse = O.sdpa_fp32(q, k, v, "HND", causal)
            c = O.compare(o, ref)
            assert c["cos"] > 0.999 and c["max_abs"] < 0.05, (causal, mode, c)
            assert float((lse - ref_lse).abs().max()) < 0.05


def test_oracle_smooth_v_removes_the_channel_offset_from_the_fp16_accumulator():
    """V with a large per-channel offset: the smoothed fp16 path (mean removed, added back after the
    normalisation) must be at least as close to exact attention as the plain fp16 accumulator."""
    g = torch.Generator().manual_seed(9)
    q = torch.randn(1, 2, 384, 64, generator=g).bfloat16()
    k = torch.randn(1, 2, 384, 64, generator=g).bfloat16()
    v = (torch.randn(1, 2, 384, 64, generator=g) + 12.0 * torch.randn(1, 2, 1, 64, generator=g)).bfloat16()
    ref, _ = O.sdpa_fp32(q, k, v, "HND", True)
    plain = O.compare(O.sageattn(q, k, v, "HND", True, "fp16"), ref)
    smooth = O.compare(O.sageattn(q, k, v, "HND", True, "fp16", smooth_v=True), ref)
    assert smooth["fro_rel"] <= plain["fro_rel"] + 1e-4 and smooth["max_abs"] <= 0.13, (plain, smooth)
    sm, vm = O.smooth_v(v, "HND")
    assert sm.dtype == torch.float16 and vm.shape == (1, 2, 64) and vm.dtype == v.dtype


def test_header_symbols_are_exported():
    hdr = open(os.path.join(ROOT, "include", "sage_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(sage_b200_[a-z0-9_]+)\s*\(", hdr)))
    assert len(declared) >= 7
    from sageattention import _capi
    lib = _capi.lib()
    for sym in declared:
        assert hasattr(lib, sym), sym
    assert set(declared) == set(_capi.EXPORTS)
    assert lib.sage_b200_version() == 100


def test_torch_operators_are_registered_natively_with_fakes():
    """The operator library loads without a GPU, registers every operator of the namespace with the
    reference's schema for the four attention operators (csrc/qattn/pybind_sm80.cpp:24-90), and the
    fake implementations return the right shapes and dtypes on meta tensors."""
    from sageattention import ops as sage_ops
    ns = torch.ops.sageattention_b200
    for name in sage_ops.ALL_OPS:
        assert hasattr(ns, name), name
    schema = str(ns.qk_int8_sv_f16_accum_f32_attn.default._schema)
    assert schema == ("sageattention_b200::qk_int8_sv_f16_accum_f32_attn(Tensor query, Tensor key, Tensor value, "
                      "Tensor(a!) output, Tensor query_scale, Tensor key_scale, int tensor_layout, bool is_causal, "
                      "float sm_scale, int blk_q, int blk_k, int warp_q, int warp_k, bool return_lse) -> Tensor")
    q = torch.empty(2, 300, 8, 128, dtype=torch.bfloat16, device="meta")          # NHD
    k = torch.empty(2, 300, 2, 128, dtype=torch.bfloat16, device="meta")
    q8, qs = ns.quant_int8(q, None, 0, 128, 32, 0, 0)
    k8, ks = ns.quant_int8(k, ns.mean_k(k, 0), 0, 64, 64, 1, 0)
    assert q8.dtype == torch.int8 and q8.shape == q.shape and qs.shape == (2, 8, 3 * 4 * 8) and ks.shape == (2, 2, 5 * 4)
    assert ns.mean_k(k, 0).shape == (2, 1, 2, 128) and ns.cast_v_f16(k, 0).dtype == torch.float16
    lse = ns.qk_int8_sv_f16_accum_f16_attn_inst_buf(q8, k8, ns.cast_v_f16(k, 0), torch.empty_like(q), qs, ks, 0, True,
                                                    0.1, 128, 64, 32, 64, True)
    assert lse.shape == (2, 8, 300) and lse.dtype == torch.float32
    out, lse, km = ns.sageattn(q, k, k, 0, True, 0.1, 128, 64, 32, 64, 0, True, 2, 0, False)
    assert out.shape == q.shape and out.is_contiguous() and lse.shape == (0,) and km.shape == (0,)
    v8, vs = ns.quant_v_fp8(k, 0)
    assert v8.dtype == torch.float8_e4m3fn and vs.shape == (2, 2, 128)


def test_public_call_traces_fullgraph_on_fake_cuda_tensors():
    """torch.compile(fullgraph=True) traces the public call (LSE, a head_dim that needs padding, GQA) and a
    function written against the per-operator path, using fake CUDA tensors: no GPU is touched, only the
    operators' fake implementations run (the reference tests the same property on a GPU,
    tests/test_sageattn_compile.py:21-31)."""
    import sageattention
    from torch._subclasses import FakeTensorMode
    ns = torch.ops.sageattention_b200

    def public(q, k, v):
        o, lse = sageattention.sageattn(q, k, v, tensor_layout="NHD", is_causal=True, return_lse=True)
        return o * 2, lse

    def per_op(q, k, v):
        km = ns.mean_k(k, 0)
        q8, qs = ns.quant_int8(q, None, 0, 128, 32, 0, 0)
        k8, ks = ns.quant_int8(k, km, 0, 64, 64, 1, 0)
        o = torch.empty_like(q)
        ns.qk_int8_sv_f16_accum_f32_attn(q8, k8, ns.cast_v_f16(v, 0), o, qs, ks, 0, True, 0.1, 128, 64, 32, 64, False)
        return o

    with FakeTensorMode():
        q = torch.empty(1, 300, 4, 80, dtype=torch.float16, device="cuda")
        k = torch.empty(1, 300, 2, 80, dtype=torch.float16, device="cuda")
        o, lse = torch.compile(public, fullgraph=True, backend="eager")(q, k, k)
        assert o.shape == q.shape and lse.shape == (1, 4, 300)
        q2 = torch.empty(2, 256, 4, 128, dtype=torch.bfloat16, device="cuda")
        assert torch.compile(per_op, fullgraph=True, backend="eager")(q2, q2, q2).shape == q2.shape
        o8 = torch.compile(lambda a, b, c: sageattention.sageattn_qk_int8_pv_fp8_cuda(a, b, c, tensor_layout="NHD"),
                           fullgraph=True, backend="eager")(q2, q2, q2)
        assert o8.shape == q2.shape


def test_argument_errors_do_not_need_a_gpu():
    from sageattention import _capi
    lib = _capi.lib()
    st = (ctypes.c_int64 * 3)(0, 0, 0)
    rc = lib.sage_b200_quant_int8(0, 0, 0, 0, 0, 1, 1, 16, 64, st, st, 128, 32, 0, 0, 0)
    assert rc == -1 and b"null pointer" in lib.sage_b200_last_error()
    rc = lib.sage_b200_mean_k(16, 16, 16, 0, 5, 1, 1, 16, 64, st, 0)
    assert rc == -1 and b"dtype" in lib.sage_b200_last_error()
    assert lib.sage_b200_mean_k_scratch_bytes(1, 64, 32768, 128) > 0
    assert lib.sage_b200_mean_k_scratch_bytes(0, 64, 32768, 128) == 0


def test_front_end_validation_matches_reference_errors():
    import sageattention
    from sageattention.core import _padded_head_dim, _sageattn_configured
    q = torch.zeros(1, 2, 16, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="CUDA"):
        sageattention.sageattn(q, q, q)
    with pytest.raises(AssertionError):
        sageattention.sageattn(q, q, q, attn_mask=torch.ones(1))
    assert [_padded_head_dim(d) for d in (32, 64, 80, 128, 129, 256)] == [64, 64, 128, 128, 256, 256]
    with pytest.raises(ValueError):
        _padded_head_dim(257)
    assert sageattention.sageattn is sageattention.sageattn_qk_int8_pv_fp16_cuda
    for name in ("sageattn_qk_int8_pv_fp8_cuda_sm90", "sageattn_varlen"):
        assert hasattr(sageattention, name)


def test_tile_table_is_total_and_consistent():
    from sageattention.tile_table import QK_CONFIGS, SUPPORTED_QK_CONFIGS, select_entry, select_qk_config
    seen = set()
    for d in (64, 128, 256):
        for causal in (False, True):
            for acc in ("fp32", "fp16", "fp16+fp32", "fp8"):
                for n in (1, 1024, 1025, 4096, 75600, 131072, 10 ** 6):
                    cfg = select_qk_config(d, causal, acc, n)
                    assert cfg in SUPPORTED_QK_CONFIGS and cfg in QK_CONFIGS
                    e = select_entry(d, causal, acc, n)
                    assert e["qk_config"] == cfg and e["q_tiles_per_cta"] in (1, 2)
                    seen.add((e["kernel"], e["q_tiles_per_cta"]))
    # the table selects among kernels: the two-level mode runs the one-tile kernel with a fold warpgroup,
    # except at head_dim 256 where only the two-tile kernel has room; the other modes run the two-tile kernel
    assert select_entry(128, True, "fp16+fp32", 32768)["kernel"] == "one_tile_fold"
    assert select_entry(128, True, "fp16+fp32", 8192)["kernel"] == "one_tile_fold"
    assert select_entry(128, True, "fp16+fp32", 6144)["kernel"] == "one_tile_persistent"
    assert select_entry(128, True, "fp16+fp32", 6145)["kernel"] == "one_tile_fold"
    assert select_entry(64, True, "fp16+fp32", 8192)["kernel"] == "one_tile_persistent"
    assert select_entry(64, True, "fp16+fp32", 8193)["kernel"] == "one_tile_fold"
    assert select_entry(128, False, "fp16+fp32", 8192)["kernel"] == "one_tile_persistent"
    assert select_entry(128, False, "fp16+fp32", 8193)["kernel"] == "one_tile_fold"
    assert select_entry(64, False, "fp16+fp32", 16384)["kernel"] == "one_tile_persistent"
    assert select_entry(64, False, "fp16+fp32", 16385)["kernel"] == "one_tile_fold"
    # ... in its persistent form (one CTA per SM walking over the tiles) up to 4096 keys
    assert select_entry(64, False, "fp16+fp32", 4096)["kernel"] == "one_tile_persistent"
    assert select_entry(128, True, "fp16+fp32", 1024)["kernel"] == "one_tile_persistent"
    assert select_entry(256, True, "fp16+fp32", 4096) == {"qk_config": (128, 64, 32, 64), "kernel": "two_tile_coupled",
                                                           "q_tiles_per_cta": 1, "seq_bucket": 2}
    assert select_entry(128, True, "fp32", 32768)["kernel"] == "two_tile"
    assert select_entry(128, True, "fp32", 32768)["q_tiles_per_cta"] == 2
    assert len(seen) >= 4


def test_output_peers_arguments_are_checked():
    import ctypes
    from sageattention import _capi as C
    L = C.lib()
    bad = (ctypes.c_int64 * 8)(*([64] * 8))
    assert L.sage_b200_set_output_peers(8, bad) != 0 and b"between 0 and 7" in L.sage_b200_last_error()
    odd = (ctypes.c_int64 * 1)(48)
    assert L.sage_b200_set_output_peers(1, odd) != 0 and b"multiple of 32" in L.sage_b200_last_error()
    assert L.sage_b200_set_output_peers(1, None) != 0
    assert L.sage_b200_set_output_peers(0, None) == 0
