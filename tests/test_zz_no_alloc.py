"""The allocation-free K-mean entry point (sage_b200_mean_k_static), called through the C ABI.

Some hosts of this library cannot allocate device memory at the point where they call it: code
inside a CUDA-graph capture, plugins given a fixed memory budget, real-time loops.  For them the
library carries its own partial-sum buffer.  The result must equal sage_b200_mean_k's exactly (same
kernels, same reduction order), also on a second call that reuses the buffer with another shape.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import pytest
import torch

from gpu_util import cuda_or_fail, make_qkv

pytestmark = pytest.mark.gpu


def _mean_with_scratch(lib, C, k, layout):
    b, h, n, d = C.bhnd(k, layout)
    km = torch.empty((b, h, d), dtype=k.dtype, device=k.device)
    nbytes = lib.sage_b200_mean_k_scratch_bytes(b, h, n, d)
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=k.device)
    C.check(lib.sage_b200_mean_k(k.data_ptr(), km.data_ptr(), scratch.data_ptr(), nbytes, C.dtype_code(k.dtype),
                                 b, h, n, d, C.bhn_strides(k, layout), C.stream_ptr(k.device)))
    return km


def _mean_static(lib, C, k, layout):
    b, h, n, d = C.bhnd(k, layout)
    km = torch.empty((b, h, d), dtype=k.dtype, device=k.device)
    C.check(lib.sage_b200_mean_k_static(k.data_ptr(), km.data_ptr(), C.dtype_code(k.dtype), b, h, n, d,
                                        C.bhn_strides(k, layout), C.stream_ptr(k.device)))
    return km


def test_static_mean_equals_scratch_mean_on_two_calls_in_a_row():
    from sageattention import _capi as C
    cuda_or_fail()
    lib = C.lib()
    assert lib.sage_b200_mean_k_static_capacity_bytes() == 2 * 1024 * 1024
    # two different shapes back to back: the second call finds the first call's partial sums in the buffer
    cases = [(2, 3, 5000, 128, torch.bfloat16, "NHD"), (1, 8, 777, 64, torch.float16, "HND")]
    for B, H, N, D, dtype, layout in cases:
        _, k, _ = make_qkv(B, H, H, N, D, dtype, layout, seed=N, k_bias=2.0)
        got = _mean_static(lib, C, k, layout)
        exp = _mean_with_scratch(lib, C, k, layout)
        torch.cuda.synchronize()
        assert torch.equal(got, exp), (B, H, N, D)
        ref = k.float().mean(dim=2 if layout == "HND" else 1).to(dtype)
        assert int((got.view(torch.int16).int() - ref.view(torch.int16).int()).abs().max()) <= 1


def test_static_mean_refuses_shapes_beyond_its_buffer():
    from sageattention import _capi as C
    cuda_or_fail()
    lib = C.lib()
    B, H, N, D = 64, 128, 128, 256                      # 8192 slabs x 256 channels of partial sums
    assert lib.sage_b200_mean_k_scratch_bytes(B, H, N, D) > lib.sage_b200_mean_k_static_capacity_bytes()
    k = torch.zeros(16, dtype=torch.float16, device="cuda")
    km = torch.zeros(16, dtype=torch.float16, device="cuda")
    st = (ctypes.c_int64 * 3)(H * N * D, N * D, D)
    rc = lib.sage_b200_mean_k_static(k.data_ptr(), km.data_ptr(), 0, B, H, N, D, st, 0)
    assert rc == -1 and b"built-in buffer" in lib.sage_b200_last_error()
