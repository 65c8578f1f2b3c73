"""Quantisation front end: K channel mean, int8 Q/K with fp32 scales, V cast.

Same call signatures and return values as the reference's Triton wrappers
(sageattention/triton/quant_per_thread.py:118-205, quant_per_block.py:81-173); the work is done
by the sm_100a kernels behind sage_b200_mean_k / sage_b200_quant_int8 / sage_b200_cast_v_f16.
"""
from __future__ import annotations

import os

import torch

from . import _capi as C

# "full": div.full.f32 like the reference's Triton kernels on a GPU; "ieee": correctly rounded
_DIV = {"full": C.DIV_FULL, "ieee": C.DIV_IEEE}


def default_div_mode() -> str:
    m = os.getenv("SAGE_B200_DIV", "full").lower()
    return m if m in _DIV else "full"


def _check_in(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError("Input tensors must be CUDA tensors.")
    if t.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported dtype: {t.dtype}")
    if t.dim() != 4 or t.stride(-1) != 1:
        raise ValueError(f"{name} must be 4-D with a contiguous last dimension.")


def _mean_k_into(k, km, tensor_layout, scratch=None):
    b, h, n, d = C.bhnd(k, tensor_layout)
    L = C.lib()
    nbytes = L.sage_b200_mean_k_scratch_bytes(b, h, n, d)
    if scratch is None or scratch.numel() * 4 < nbytes:
        scratch = torch.empty(max(nbytes, 4) // 4, dtype=torch.float32, device=k.device)
    with torch.cuda.device(k.device):
        C.check(L.sage_b200_mean_k(k.data_ptr(), km.data_ptr(), scratch.data_ptr(), scratch.numel() * 4,
                                   C.dtype_code(k.dtype), b, h, n, d, C.bhn_strides(k, tensor_layout),
                                   C.stream_ptr(k.device)))
    return scratch


def mean_k(k: torch.Tensor, tensor_layout: str = "HND") -> torch.Tensor:
    """k.mean over the sequence, keepdim, in k's dtype (reference: cuda_attn.py:167-170)."""
    _check_in(k, "k")
    b, h, n, d = C.bhnd(k, tensor_layout)
    shape = (b, h, 1, d) if tensor_layout == "HND" else (b, 1, h, d)
    km = torch.empty(shape, dtype=k.dtype, device=k.device)
    _mean_k_into(k, km, tensor_layout)
    return km


def _groups(n, blk, warp, kind):
    blocks = -(-n // blk)
    if kind == C.GROUP_Q_THREAD:
        return blocks * (blk // warp) * 8
    if kind == C.GROUP_K_THREAD:
        return blocks * (blk // warp) * 4
    return blocks


def _quant_into(x, mean, out, scale, blk, warp, kind, tensor_layout, div):
    b, h, n, d = C.bhnd(x, tensor_layout)
    with torch.cuda.device(x.device):
        C.check(C.lib().sage_b200_quant_int8(
            x.data_ptr(), 0 if mean is None else mean.data_ptr(), out.data_ptr(), scale.data_ptr(),
            C.dtype_code(x.dtype), b, h, n, d, C.bhn_strides(x, tensor_layout), C.bhn_strides(out, tensor_layout),
            blk, warp, kind, _DIV[div], C.stream_ptr(x.device)))


def _quant_one(x, mean, blk, warp, kind, tensor_layout, div):
    b, h, n, d = C.bhnd(x, tensor_layout)
    out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty((b, h, _groups(n, blk, warp, kind)), dtype=torch.float32, device=x.device)
    if mean is not None:
        if mean.dtype != x.dtype or mean.numel() != b * h * d:
            raise ValueError("km must have k's dtype and one value per (batch, head, channel).")
        mean = mean.contiguous()
    _quant_into(x, mean, out, scale, blk, warp, kind, tensor_layout, div)
    return out, scale


# K is read twice (mean, then quantise).  The C call can do both per L2-sized slice of heads so that
# the second read hits L2, but on B200 the extra launches cost more than the saved HBM traffic
# (0.32 ms unsliced vs 0.46 ms in 64 MiB slices at 64 x 32768 x 128), so the default is one slice.
_L2_SLICE_BYTES = 0


def smooth_quant_k(k, blk, warp, kind, tensor_layout="HND", div=None):
    """(km, k_int8, k_scale): channel mean of K and int8 quantisation of K - mean in one C call."""
    _check_in(k, "k")
    div = div or default_div_mode()
    b, h, n, d = C.bhnd(k, tensor_layout)
    km = torch.empty((b, h, 1, d) if tensor_layout == "HND" else (b, 1, h, d), dtype=k.dtype, device=k.device)
    k8 = torch.empty(k.shape, dtype=torch.int8, device=k.device)
    ks = torch.empty((b, h, _groups(n, blk, warp, kind)), dtype=torch.float32, device=k.device)
    L = C.lib()
    nbytes = L.sage_b200_smooth_quant_k_scratch_bytes(b, h, n, d, _L2_SLICE_BYTES)
    scratch = torch.empty(max(nbytes, 4) // 4, dtype=torch.float32, device=k.device)
    with torch.cuda.device(k.device):
        C.check(L.sage_b200_smooth_quant_k(
            k.data_ptr(), km.data_ptr(), k8.data_ptr(), ks.data_ptr(), scratch.data_ptr(), scratch.numel() * 4,
            C.dtype_code(k.dtype), b, h, n, d, C.bhn_strides(k, tensor_layout), C.bhn_strides(k8, tensor_layout),
            blk, warp, kind, _DIV[div], _L2_SLICE_BYTES, C.stream_ptr(k.device)))
    return km, k8, ks


def per_thread_int8(q, k, km=None, BLKQ=128, WARPQ=32, BLKK=64, WARPK=64, tensor_layout="HND", div=None):
    """(q_int8, q_scale, k_int8, k_scale) with the reference's per-thread scale grouping."""
    _check_in(q, "q")
    _check_in(k, "k")
    div = div or default_div_mode()
    q8, qs = _quant_one(q, None, BLKQ, WARPQ, C.GROUP_Q_THREAD, tensor_layout, div)
    k8, ks = _quant_one(k, km, BLKK, WARPK, C.GROUP_K_THREAD, tensor_layout, div)
    return q8, qs, k8, ks


def per_block_int8(q, k, km=None, BLKQ=128, BLKK=64, tensor_layout="HND", div=None):
    """(q_int8, q_scale, k_int8, k_scale) with one scale per BLKQ x D / BLKK x D tile."""
    _check_in(q, "q")
    _check_in(k, "k")
    div = div or default_div_mode()
    q8, qs = _quant_one(q, None, BLKQ, BLKQ, C.GROUP_BLOCK, tensor_layout, div)
    k8, ks = _quant_one(k, km, BLKK, BLKK, C.GROUP_BLOCK, tensor_layout, div)
    return q8, qs, k8, ks


def cast_v_fp16(v: torch.Tensor, tensor_layout: str = "HND") -> torch.Tensor:
    """v.to(torch.float16) (reference: cuda_attn.py:195); fp16 input with TMA-friendly strides is
    returned as is."""
    _check_in(v, "v")
    if v.dtype == torch.float16 and v.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in v.stride()[:3]):
        return v
    b, h, n, d = C.bhnd(v, tensor_layout)
    out = torch.empty(v.shape, dtype=torch.float16, device=v.device)
    with torch.cuda.device(v.device):
        C.check(C.lib().sage_b200_cast_v_f16(
            v.data_ptr(), out.data_ptr(), C.dtype_code(v.dtype), b, h, n, d,
            C.bhn_strides(v, tensor_layout), C.bhn_strides(out, tensor_layout), C.stream_ptr(v.device)))
    return out


def smooth_v_fp16(v: torch.Tensor, tensor_layout: str = "HND"):
    """(smoothed_v, vm): vm = v.mean over the sequence, (batch, heads, head_dim) in v's dtype, and
    (v - vm).to(float16) with the difference rounded to v's dtype first (reference: cuda_attn.py:209-211)."""
    _check_in(v, "v")
    b, h, n, d = C.bhnd(v, tensor_layout)
    vm4 = mean_k(v, tensor_layout)                      # the channel-mean kernels do not care which tensor it is
    vm = vm4.view(b, h, d)
    out = torch.empty(v.shape, dtype=torch.float16, device=v.device)
    with torch.cuda.device(v.device):
        C.check(C.lib().sage_b200_smooth_v_f16(
            v.data_ptr(), vm.data_ptr(), out.data_ptr(), C.dtype_code(v.dtype), b, h, n, d,
            C.bhn_strides(v, tensor_layout), C.bhn_strides(out, tensor_layout), C.stream_ptr(v.device)))
    return out, vm


def quant_v_fp8(v: torch.Tensor, tensor_layout: str = "HND"):
    """(v_fp8, v_scale): V in fp8 e4m3 with one fp32 scale per (batch, head, channel),
    scale = max|v| over the sequence / 448.  v_fp8 keeps v's shape and dimension order
    (dtype torch.float8_e4m3fn), v_scale is (batch, heads, head_dim)."""
    _check_in(v, "v")
    b, h, n, d = C.bhnd(v, tensor_layout)
    out = torch.empty(v.shape, dtype=torch.uint8, device=v.device)
    v_scale = torch.empty((b, h, d), dtype=torch.float32, device=v.device)
    L = C.lib()
    nbytes = L.sage_b200_quant_v_fp8_scratch_bytes(b, h, n, d)
    scratch = torch.empty(max(nbytes, 4) // 4, dtype=torch.float32, device=v.device)
    with torch.cuda.device(v.device):
        C.check(L.sage_b200_quant_v_fp8(v.data_ptr(), out.data_ptr(), v_scale.data_ptr(), scratch.data_ptr(),
                                        scratch.numel() * 4, C.dtype_code(v.dtype), b, h, n, d,
                                        C.bhn_strides(v, tensor_layout), C.bhn_strides(out, tensor_layout),
                                        C.stream_ptr(v.device)))
    return out.view(torch.float8_e4m3fn), v_scale
