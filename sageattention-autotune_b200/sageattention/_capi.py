"""ctypes binding of libsage_b200.so (declared in include/sage_b200.h).

This is the only place the Python package touches native code.  There is no fallback: if the
library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# SAGE_B200_LIB names another build of the same library (kernel experiments); normally unset
_LIB_PATH = os.environ.get("SAGE_B200_LIB") or os.path.join(_HERE, "libsage_b200.so")

F16, BF16 = 0, 1
GROUP_Q_THREAD, GROUP_K_THREAD, GROUP_BLOCK = 0, 1, 2
DIV_FULL, DIV_IEEE = 0, 1
GRAN_PER_THREAD, GRAN_PER_BLOCK = 0, 1
PV_F32, PV_F16, PV_F16_F32, PV_F8 = 0, 1, 2, 3

EXPORTS = (
    "sage_b200_version", "sage_b200_last_error", "sage_b200_mean_k_scratch_bytes", "sage_b200_mean_k",
    "sage_b200_mean_k_static_capacity_bytes", "sage_b200_mean_k_static",
    "sage_b200_quant_int8", "sage_b200_smooth_quant_k_scratch_bytes", "sage_b200_smooth_quant_k",
    "sage_b200_cast_v_f16", "sage_b200_attn_fwd", "sage_b200_quant_v_fp8_scratch_bytes", "sage_b200_quant_v_fp8",
    "sage_b200_attn_fwd_fp8", "sage_b200_smooth_v_f16", "sage_b200_attn_fwd_fuse_v_mean",
    "sage_b200_sageattn_workspace_bytes", "sage_b200_sageattn", "sage_b200_set_wait_budget", "sage_b200_launch_count", "sage_b200_tile_lookup",
    "sage_b200_peer_alloc", "sage_b200_peer_open", "sage_b200_peer_close", "sage_b200_peer_free",
    "sage_b200_set_output_peers",
)

_lib = None
_I64x3 = ctypes.c_int64 * 3


class SageB200Error(RuntimeError):
    pass


class TileEntry(ctypes.Structure):
    """sage_b200_tile_entry of include/sage_b200.h"""
    _fields_ = [("blk_q", ctypes.c_int), ("blk_k", ctypes.c_int), ("warp_q", ctypes.c_int), ("warp_k", ctypes.c_int),
                ("kernel", ctypes.c_int), ("q_tiles_per_cta", ctypes.c_int), ("seq_bucket", ctypes.c_int)]


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(
                f"{_LIB_PATH} is missing: build it with `python sageattention-autotune_b200/build.py` "
                "(there is no non-CUDA fallback)")
        L = ctypes.CDLL(_LIB_PATH)
        vp, i, i64p, f = ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int64), ctypes.c_float
        L.sage_b200_version.restype = i
        L.sage_b200_last_error.restype = ctypes.c_char_p
        L.sage_b200_mean_k_scratch_bytes.restype = ctypes.c_size_t
        L.sage_b200_mean_k_scratch_bytes.argtypes = [i, i, i, i]
        L.sage_b200_mean_k.restype = i
        L.sage_b200_mean_k.argtypes = [vp, vp, vp, ctypes.c_size_t, i, i, i, i, i, i64p, vp]
        L.sage_b200_mean_k_static_capacity_bytes.restype = ctypes.c_size_t
        L.sage_b200_mean_k_static.restype = i
        L.sage_b200_mean_k_static.argtypes = [vp, vp, i, i, i, i, i, i64p, vp]
        L.sage_b200_quant_int8.restype = i
        L.sage_b200_quant_int8.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i64p, i64p, i, i, i, i, vp]
        L.sage_b200_smooth_quant_k_scratch_bytes.restype = ctypes.c_size_t
        L.sage_b200_smooth_quant_k_scratch_bytes.argtypes = [i, i, i, i, ctypes.c_size_t]
        L.sage_b200_smooth_quant_k.restype = i
        L.sage_b200_smooth_quant_k.argtypes = [vp, vp, vp, vp, vp, ctypes.c_size_t, i, i, i, i, i, i64p, i64p,
                                               i, i, i, i, ctypes.c_size_t, vp]
        L.sage_b200_cast_v_f16.restype = i
        L.sage_b200_cast_v_f16.argtypes = [vp, vp, i, i, i, i, i, i64p, i64p, vp]
        L.sage_b200_attn_fwd.restype = i
        L.sage_b200_attn_fwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i,
                                         i64p, i64p, i64p, i64p, i, f, i, i, i, i, i, i, vp]
        L.sage_b200_quant_v_fp8_scratch_bytes.restype = ctypes.c_size_t
        L.sage_b200_quant_v_fp8_scratch_bytes.argtypes = [i, i, i, i]
        L.sage_b200_quant_v_fp8.restype = i
        L.sage_b200_quant_v_fp8.argtypes = [vp, vp, vp, vp, ctypes.c_size_t, i, i, i, i, i, i64p, i64p, vp]
        L.sage_b200_attn_fwd_fp8.restype = i
        L.sage_b200_attn_fwd_fp8.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i,
                                             i64p, i64p, i64p, i64p, i, f, i, i, i, i, i, vp]
        L.sage_b200_smooth_v_f16.restype = i
        L.sage_b200_smooth_v_f16.argtypes = [vp, vp, vp, i, i, i, i, i, i64p, i64p, vp]
        L.sage_b200_attn_fwd_fuse_v_mean.restype = i
        L.sage_b200_attn_fwd_fuse_v_mean.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i,
                                                     i64p, i64p, i64p, i64p, i, f, i, i, i, i, i, vp]
        L.sage_b200_sageattn_workspace_bytes.restype = ctypes.c_size_t
        L.sage_b200_sageattn_workspace_bytes.argtypes = [i] * 14
        L.sage_b200_sageattn.restype = i
        L.sage_b200_sageattn.argtypes = [vp, vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp, i, i, i, i, i, i, i,
                                         i64p, i64p, i64p, i64p, i, f, i, i, i, i, i, i, i, i, vp]
        L.sage_b200_tile_lookup.restype = i
        L.sage_b200_tile_lookup.argtypes = [i, i, i, i, ctypes.POINTER(TileEntry)]
        L.sage_b200_launch_count.restype = ctypes.c_ulonglong
        L.sage_b200_set_wait_budget.restype = ctypes.c_longlong
        L.sage_b200_set_wait_budget.argtypes = [ctypes.c_longlong]
        L.sage_b200_peer_alloc.restype = i
        L.sage_b200_peer_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(vp), ctypes.c_char_p]
        L.sage_b200_peer_open.restype = i
        L.sage_b200_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        L.sage_b200_peer_close.restype = i
        L.sage_b200_peer_close.argtypes = [vp]
        L.sage_b200_peer_free.restype = i
        L.sage_b200_peer_free.argtypes = [vp]
        L.sage_b200_set_output_peers.restype = i
        L.sage_b200_set_output_peers.argtypes = [i, i64p]
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise SageB200Error(f"sage_b200 error {rc}: {lib().sage_b200_last_error().decode()}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return F16
    if dt == torch.bfloat16:
        return BF16
    raise ValueError(f"Unsupported dtype: {dt}")


def bhn_strides(t: torch.Tensor, tensor_layout: str):
    """Element strides in (batch, head, seq) order for either layout."""
    if tensor_layout == "HND":
        return _I64x3(t.stride(0), t.stride(1), t.stride(2))
    return _I64x3(t.stride(0), t.stride(2), t.stride(1))


def bhnd(t: torch.Tensor, tensor_layout: str):
    if tensor_layout == "HND":
        b, h, n, d = t.shape
    elif tensor_layout == "NHD":
        b, n, h, d = t.shape
    else:
        raise ValueError("tensor_layout must be 'NHD' or 'HND'.")
    return b, h, n, d


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
