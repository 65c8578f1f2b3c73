"""The natively registered torch operators (namespace sageattention_b200) on the GPU.

They are the inner boundary a caller of the reference binds to: torch.ops.sageattention_qattn_sm80.*
(csrc/qattn/pybind_sm80.cpp:24-98) with the same names and argument lists.  Each operator must give
the bits of the ctypes route, and torch.compile(fullgraph=True) must trace functions that use them.
"""
import pytest
import torch

from gpu_util import cuda_or_fail, make_qkv, reference_ops

pytestmark = pytest.mark.gpu
CFG = (128, 64, 32, 64)


def _ops():
    import sageattention  # noqa: F401  (loads the operator library)
    return torch.ops.sageattention_b200


@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_front_end_operators_equal_the_ctypes_route(layout):
    from sageattention import quant
    cuda_or_fail()
    ops = _ops()
    code = 1 if layout == "HND" else 0
    q, k, v = make_qkv(2, 4, 2, 777, 128, torch.bfloat16, layout, seed=5, k_bias=1.0)
    km = ops.mean_k(k, code)
    assert torch.equal(km, quant.mean_k(k, layout))
    q8, qs, k8, ks = quant.per_thread_int8(q, k, km, tensor_layout=layout)
    q8o, qso = ops.quant_int8(q, None, code, 128, 32, 0, 0)
    k8o, kso = ops.quant_int8(k, km, code, 64, 64, 1, 0)
    assert torch.equal(q8o, q8) and torch.equal(qso, qs) and torch.equal(k8o, k8) and torch.equal(kso, ks)
    b8, bs = ops.quant_int8(k, km, code, 64, 64, 2, 0)
    assert torch.equal(b8, quant.per_block_int8(q, k, km, 128, 64, layout)[2])
    assert torch.equal(ops.cast_v_f16(v, code), v.to(torch.float16))
    v8, vs = ops.quant_v_fp8(v, code)
    e8, es = quant.quant_v_fp8(v, layout)
    assert torch.equal(v8.view(torch.uint8), e8.view(torch.uint8)) and torch.equal(vs, es)


@pytest.mark.parametrize("mode,op", [("fp32", "qk_int8_sv_f16_accum_f32_attn"),
                                      ("fp16+fp32", "qk_int8_sv_f16_accum_f16_attn_inst_buf"),
                                      ("fp16", "qk_int8_sv_f16_accum_f16_attn")])
def test_attention_operators_take_the_reference_argument_list(mode, op):
    """The same positional call goes to torch.ops.sageattention_qattn_sm80.<op> (the reference's kernels,
    rebuilt) and to torch.ops.sageattention_b200.<op>; the latter equals the ctypes route bit for bit."""
    from sageattention import quant
    from sageattention.core import attn_fwd_quantized
    cuda_or_fail()
    ops = _ops()
    q, k, v = make_qkv(1, 4, 2, 1000, 128, torch.float16, "HND", seed=6, k_bias=1.0)
    km = quant.mean_k(k)
    q8, qs, k8, ks = quant.per_thread_int8(q, k, km)
    out = torch.empty_like(q)
    args = (q8, k8, v, out, qs, ks, 1, True, 128 ** -0.5, *CFG, True)
    lse = getattr(ops, op)(*args)
    exp = torch.empty_like(q)
    exp_lse = attn_fwd_quantized(q8, k8, v, exp, qs, ks, "HND", True, 128 ** -0.5, CFG, mode, True)
    torch.cuda.synchronize()
    assert lse.shape == (1, 4, 1000) and torch.equal(out, exp) and torch.equal(lse, exp_lse)
    ref = reference_ops()
    if ref is not None:
        ref_out = torch.empty_like(q)
        getattr(ref, op)(*args[:3], ref_out, *args[4:-1], False)
        torch.cuda.synchronize()
        a, b = out.float().flatten(), ref_out.float().flatten()
        assert float(torch.dot(a, b) / (a.norm() * b.norm())) >= 0.9995 and float((a - b).abs().max()) <= 2e-2


def test_operator_argument_errors_raise():
    """A bad argument (fp32 V, an unknown layout, a grouping no kernel is built for, a 3-D tensor) raises
    RuntimeError through torch's stable ABI, as the reference's STD_TORCH_CHECKs do; no kernel runs.
    (This needs the operator library to share the C++ run time with torch: a build that links a private
    libstdc++ kills the process here instead.)"""
    cuda_or_fail()
    ops = _ops()
    q8 = torch.zeros(1, 2, 64, 128, dtype=torch.int8, device="cuda")
    v = torch.zeros(1, 2, 64, 128, dtype=torch.float16, device="cuda")
    out = torch.zeros_like(v)
    s = torch.ones(1, 2, 16, device="cuda")
    op = ops.qk_int8_sv_f16_accum_f32_attn
    with pytest.raises(RuntimeError, match="fp16"):
        op(q8, q8, v.float(), out, s, s, 1, True, 0.1, *CFG, False)
    with pytest.raises(RuntimeError, match="tensor_layout"):
        op(q8, q8, v, out, s, s, 7, True, 0.1, *CFG, False)
    with pytest.raises(RuntimeError, match="warp_k"):
        op(q8, q8, v, out, s, s, 1, True, 0.1, 128, 64, 32, 32, False)
    with pytest.raises(RuntimeError):
        ops.mean_k(v[0], 1)
    with pytest.raises(RuntimeError):
        ops.quant_int8(v, None, 1, 128, 256, 0, 0)
    torch.cuda.synchronize()
    assert bool((out == 0).all())


def test_whole_call_operator_and_compile_fullgraph():
    import sageattention
    cuda_or_fail()
    ops = _ops()
    q, k, v = make_qkv(1, 4, 2, 640, 128, torch.bfloat16, "NHD", seed=7, k_bias=1.0)
    out, lse, km = ops.sageattn(q, k, v, 0, True, 128 ** -0.5, *CFG, 0, True, 2, 0, True)
    exp, exp_lse = sageattention.sageattn(q, k, v, tensor_layout="NHD", is_causal=True, pv_accum_dtype="fp16+fp32",
                                          return_lse=True)
    torch.cuda.synchronize()
    assert torch.equal(out, exp) and km.shape == (1, 1, 2, 128) and lse.shape == (1, 4, 640)

    # a function written against the per-operator path, as a caller of the reference's operators would
    def per_op(q, k, v):
        km = ops.mean_k(k, 0)
        q8, qs = ops.quant_int8(q, None, 0, 128, 32, 0, 0)
        k8, ks = ops.quant_int8(k, km, 0, 64, 64, 1, 0)
        o = torch.empty_like(q)
        ops.qk_int8_sv_f16_accum_f32_attn(q8, k8, ops.cast_v_f16(v, 0), o, qs, ks, 0, True, 128 ** -0.5, *CFG, False)
        return o * 2.0

    got = torch.compile(per_op, fullgraph=True, backend="aot_eager")(q, k, v)
    assert torch.allclose(got.float(), per_op(q, k, v).float(), atol=1e-3)

    # the public call, with the LSE, a head_dim that needs padding and a non-contiguous q
    def public(q, k, v):
        o, l = sageattention.sageattn(q, k, v, tensor_layout="NHD", is_causal=True, return_lse=True)
        return o + 1.0, l

    qp, kp, vp = make_qkv(1, 4, 4, 300, 80, torch.float16, "NHD", seed=8)
    qn = torch.empty(1, 300, 4, 96, dtype=torch.float16, device=qp.device)[..., :80]
    qn.copy_(qp)
    assert not qn.is_contiguous()
    got_o, got_l = torch.compile(public, fullgraph=True, backend="aot_eager")(qn, kp, vp)
    exp_o, exp_l = public(qn, kp, vp)
    assert got_o.shape == exp_o.shape and got_o.stride() == exp_o.stride()
    assert torch.allclose(got_o.float(), exp_o.float(), atol=1e-3) and torch.allclose(got_l, exp_l, atol=1e-3)
