"""The attention epilogue's extra copies of the output (sage_b200_set_output_peers) on one GPU.

On a node the copies live in other GPUs' memory; the kernel only sees byte offsets, so here they are more
buffers on the same GPU.  Every copy must equal the local output to the bit, for every kernel of the
tile table, and the rows a CTA gives up on must read as NaN in every copy.
"""
import ctypes

import pytest
import torch

from gpu_util import cuda_or_fail, make_qkv

pytestmark = pytest.mark.gpu


def _with_copies(fn, q, copies, **kw):
    """run fn(q, ...) with its output in buffers[0] and `copies` more copies behind it"""
    from sageattention import _capi as C
    from sageattention.core import output_into
    buffers = torch.zeros((copies + 1,) + tuple(q.shape), dtype=q.dtype, device=q.device)
    base = buffers[0].data_ptr()
    offsets = (ctypes.c_int64 * copies)(*[buffers[i + 1].data_ptr() - base for i in range(copies)])
    C.check(C.lib().sage_b200_set_output_peers(copies, offsets))
    try:
        with output_into(buffers[0]):
            out = fn(q, **kw)
    finally:
        C.check(C.lib().sage_b200_set_output_peers(0, None))
    torch.cuda.synchronize()
    assert out.data_ptr() == base
    return buffers


@pytest.mark.parametrize("mode,n,d,causal,layout,dtype,copies", [
    ("fp16+fp32", 1500, 128, True, "HND", torch.float16, 1),     # persistent one-tile kernel
    ("fp16+fp32", 1000, 64, False, "NHD", torch.bfloat16, 3),
    ("fp16+fp32", 5000, 128, True, "HND", torch.bfloat16, 7),    # one CTA per tile
    ("fp32", 1500, 128, True, "NHD", torch.float16, 2),          # two-tile kernel
    ("fp32", 900, 256, False, "HND", torch.bfloat16, 1),
    ("fp16", 1100, 64, True, "HND", torch.float16, 1),
])
def test_every_copy_of_the_output_equals_the_local_one(mode, n, d, causal, layout, dtype, copies):
    import sageattention
    cuda_or_fail()
    q, k, v = make_qkv(2, 4, 2, n, d, dtype, layout, seed=17, k_bias=1.0)
    kw = dict(tensor_layout=layout, is_causal=causal, pv_accum_dtype=mode)
    plain = sageattention.sageattn(q, k, v, **kw)
    buffers = _with_copies(lambda q_, **kw_: sageattention.sageattn(q_, k, v, **kw_), q, copies, **kw)
    for i in range(copies + 1):
        assert torch.equal(buffers[i], plain), f"copy {i}"
    # the set is cleared: the next call writes one output only
    again = sageattention.sageattn(q, k, v, **kw)
    assert torch.equal(again, plain)


def test_fp8_and_smoothed_v_kernels_write_the_copies_too():
    import sageattention
    cuda_or_fail()
    q, k, v = make_qkv(1, 4, 4, 1300, 128, torch.float16, "HND", seed=19, k_bias=1.0)
    for fn, kw in ((sageattention.sageattn_qk_int8_pv_fp8_cuda, dict(is_causal=True)),
                   (sageattention.sageattn, dict(is_causal=False, pv_accum_dtype="fp16", smooth_v=True))):
        plain = fn(q, k, v, **kw)
        buffers = _with_copies(lambda q_, **kw_: fn(q_, k, v, **kw_), q, 2, **kw)
        for i in range(3):
            assert torch.equal(buffers[i], plain)


def test_rows_given_up_read_as_nan_in_every_copy(monkeypatch):
    import sageattention
    from sageattention import _capi as C
    from sageattention import core
    cuda_or_fail()
    q, k, v = make_qkv(1, 4, 2, 700, 128, torch.float16, "HND", seed=81, k_bias=1.0)
    kw = dict(tensor_layout="HND", is_causal=True, pv_accum_dtype="fp16+fp32")
    monkeypatch.setenv("SAGE_B200_CHECK", "0")
    C.lib().sage_b200_set_wait_budget(1)
    try:
        buffers = _with_copies(lambda q_, **kw_: sageattention.sageattn(q_, k, v, **kw_), q, 2, **kw)
    finally:
        C.lib().sage_b200_set_wait_budget(0)
    nan0 = torch.isnan(buffers[0].float())
    assert bool(nan0.any())
    for i in (1, 2):
        assert torch.equal(torch.isnan(buffers[i].float()), nan0)
    with pytest.raises(C.SageB200Error):
        core.check_device_status(q.device)
