"""Public API: drop-in for `sageattention` of woct0rdho/sageattention-autotune.

Mirrors sageattention/core.py:6-21 (names and placeholders) and sageattention/cuda_attn.py:44-274
(argument checks, head-dim padding, K smoothing, quantisation, accumulate-mode dispatch, LSE
fix-up) on top of the sm_100a kernels.  Differences from the reference, all additive:
`sm_scale` keyword (default head_dim**-0.5), `qk_quant_gran` keyword ("per_thread" is what the
reference's CUDA backend uses, "per_block" what its Triton backend uses), a working `return_lse`.
"""
from __future__ import annotations

import os
import warnings
from typing import Optional

import torch
import torch.nn.functional as F

from . import _capi as C
from . import ops as _ops          # loads the operator library and registers the fakes
from . import quant as Q
from .quant import cast_v_fp16, mean_k, per_block_int8, per_thread_int8
from .tile_table import SUPPORTED_QK_CONFIGS, select_qk_config

LOG2_E = 1.44269504088896340736

DEFAULT_PV_ACCUM_DTYPE = os.getenv("SAGEATTN_DEFAULT_PV_ACCUM_DTYPE", "fp32").lower()
if DEFAULT_PV_ACCUM_DTYPE not in ("fp32", "fp16", "fp16+fp32"):
    DEFAULT_PV_ACCUM_DTYPE = "fp32"

_PV_CODE = {"fp32": C.PV_F32, "fp16": C.PV_F16, "fp16+fp32": C.PV_F16_F32}
_FP8_PV = "fp8"      # internal selector of the e4m3 P.V kernel


import contextlib
import threading

_into = threading.local()


@contextlib.contextmanager
def output_into(buffer: torch.Tensor):
    """Inside the block, the attention calls of this thread write their output into `buffer` (same
    shape and dtype as q, head_dim a supported size so that nothing is padded) instead of a fresh
    tensor, and return it.  Used by the head-sharded call, whose output lives in memory that the
    other GPUs of the node have mapped."""
    previous = getattr(_into, "buffer", None)
    _into.buffer = buffer
    try:
        yield
    finally:
        _into.buffer = previous


def _new_output(q: torch.Tensor, head_dim: int) -> torch.Tensor:
    buffer = getattr(_into, "buffer", None)
    if buffer is None:
        return torch.empty(q.size(), dtype=q.dtype, device=q.device)
    if buffer.shape != q.shape or buffer.dtype != q.dtype or buffer.device != q.device or head_dim != q.size(-1):
        raise ValueError("output_into: the buffer must have q's shape (an unpadded head_dim), dtype and device")
    if buffer.stride(-1) != 1:
        raise ValueError("output_into: the last dimension of the buffer must be contiguous")
    return buffer


# When set to a list, (label, start_event, end_event) is appended around each group of kernel
# launches, so that callers (the benchmark) can time the attention kernel alone inside a full call.
_profile = None


class _Timed:
    def __init__(self, label):
        self.label = label

    def __enter__(self):
        if _profile is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if _profile is not None:
            self.end.record()
            _profile.append((self.label, self.start, self.end))
        return False


def _check_status_enabled() -> bool:
    return os.getenv("SAGE_B200_CHECK", "0").lower() in ("1", "true", "yes", "on")


# Device-side failures (a bounded wait inside the attention kernel ran out) are reported through a
# status word.  Every launch gets one: four int32 per device in pinned host memory, which the GPU
# writes through its mapped address and the host reads without synchronising.  The word is looked
# at before the next launch on that device (so a failure surfaces one call late, never silently)
# and by check_device_status(); with SAGE_B200_CHECK=1 every call synchronises and checks at once.
_status_words = {}


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(idx)
    if word is None:
        word = torch.zeros(4, dtype=torch.int32).pin_memory()
        _status_words[idx] = word
    return word


def _raise_if_failed(word: torch.Tensor, when: str) -> None:
    code = int(word[0])
    if code != 0:
        cta = tuple(int(x) for x in word[1:])
        word.zero_()
        raise C.SageB200Error(f"{when} attention launch gave up waiting (code {code}) in CTA {cta}; "
                              "its output rows read as NaN")


def check_device_status(device=None, synchronize: bool = True) -> None:
    """Raise SageB200Error if an attention launch on `device` reported a failure since the last check."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if synchronize:
        torch.cuda.synchronize(device)
    _raise_if_failed(_status_word(device), "an earlier")


def _launch_status(device: torch.device) -> torch.Tensor:
    word = _status_word(device)
    _raise_if_failed(word, "an earlier")
    return word


def _after_launch(device: torch.device, word: torch.Tensor) -> None:
    if _check_status_enabled() and not torch.cuda.is_current_stream_capturing():
        torch.cuda.synchronize(device)
        _raise_if_failed(word, "the")


def _padded_head_dim(head_dim: int) -> int:
    for edge in (64, 128, 256):
        if head_dim <= edge:
            return edge
    raise ValueError(f"Unsupported head_dim: {head_dim}")


def _pad_qkv(q, k, v):
    head_dim = q.size(-1)
    pad_to = _padded_head_dim(head_dim)
    if pad_to == head_dim:
        return head_dim, q, k, v
    pad = (0, pad_to - head_dim)
    return head_dim, F.pad(q, pad), F.pad(k, pad), F.pad(v, pad)


def _lse_correction(q, km, tensor_layout):
    """q . km^T per query row, fp32, with GQA broadcast (reference: utils.py:39-49)."""
    h_dim = 1 if tensor_layout == "HND" else 2
    rep = q.size(h_dim) // km.size(h_dim)
    if rep > 1:
        km = torch.repeat_interleave(km, rep, dim=h_dim)
    if tensor_layout == "NHD":
        corr = torch.matmul(q.transpose(1, 2), km.permute(0, 2, 3, 1)).squeeze(-1)
    else:
        corr = torch.matmul(q, km.transpose(2, 3)).squeeze(-1)
    return corr.to(torch.float32)


def attn_fwd_quantized(q_int8, k_int8, v_fp16, output, q_scale, k_scale, tensor_layout, is_causal, sm_scale,
                       qk_config, pv_accum_dtype="fp32", return_lse=False, granularity="per_thread", v_scale=None,
                       v_mean=None):
    """The attention core on pre-quantised tensors; the counterpart of
    torch.ops.sageattention_qattn_sm80.qk_int8_sv_f16_accum_*_attn (csrc/qattn/pybind_sm80.cpp:24-98).
    Writes `output` in place and returns the base-2 LSE ((0,)-shaped when not requested).
    `v_mean` ((batch, kv_heads, head_dim), output dtype) selects the fp16 accumulator with the mean of a
    smoothed V added back (..._accum_f16_fuse_v_mean_attn)."""
    fp8 = v_scale is not None
    if v_mean is not None and (fp8 or pv_accum_dtype != "fp16"):
        raise ValueError("v_mean goes with pv_accum_dtype='fp16' only.")
    if not fp8 and pv_accum_dtype not in _PV_CODE:
        raise ValueError("pv_accum_dtype must be 'fp32', 'fp16', or 'fp16+fp32'.")
    b, hq, nq, d = C.bhnd(q_int8, tensor_layout)
    _, hkv, nk, _ = C.bhnd(k_int8, tensor_layout)
    blk_q, blk_k, warp_q, warp_k = qk_config
    dev = q_int8.device
    lse = torch.empty((b, hq, nq) if return_lse else (0,), dtype=torch.float32, device=dev)
    status = _launch_status(dev)
    gran = C.GRAN_PER_THREAD if granularity == "per_thread" else C.GRAN_PER_BLOCK
    with torch.cuda.device(dev):
        if fp8:
            C.check(C.lib().sage_b200_attn_fwd_fp8(
                q_int8.data_ptr(), k_int8.data_ptr(), v_fp16.data_ptr(), v_scale.data_ptr(), output.data_ptr(),
                q_scale.data_ptr(), k_scale.data_ptr(), lse.data_ptr() if return_lse else 0,
                status.data_ptr(), C.dtype_code(output.dtype), b, hq, hkv, nq, nk, d,
                C.bhn_strides(q_int8, tensor_layout), C.bhn_strides(k_int8, tensor_layout),
                C.bhn_strides(v_fp16, tensor_layout), C.bhn_strides(output, tensor_layout),
                1 if is_causal else 0, float(sm_scale), blk_q, blk_k, warp_q, warp_k, gran, C.stream_ptr(dev)))
        elif v_mean is not None:
            v_mean = v_mean.to(output.dtype).contiguous()
            C.check(C.lib().sage_b200_attn_fwd_fuse_v_mean(
                q_int8.data_ptr(), k_int8.data_ptr(), v_fp16.data_ptr(), v_mean.data_ptr(), output.data_ptr(),
                q_scale.data_ptr(), k_scale.data_ptr(), lse.data_ptr() if return_lse else 0,
                status.data_ptr(), C.dtype_code(output.dtype), b, hq, hkv, nq, nk, d,
                C.bhn_strides(q_int8, tensor_layout), C.bhn_strides(k_int8, tensor_layout),
                C.bhn_strides(v_fp16, tensor_layout), C.bhn_strides(output, tensor_layout),
                1 if is_causal else 0, float(sm_scale), blk_q, blk_k, warp_q, warp_k, gran, C.stream_ptr(dev)))
        else:
            C.check(C.lib().sage_b200_attn_fwd(
                q_int8.data_ptr(), k_int8.data_ptr(), v_fp16.data_ptr(), output.data_ptr(),
                q_scale.data_ptr(), k_scale.data_ptr(), lse.data_ptr() if return_lse else 0,
                status.data_ptr(), C.dtype_code(output.dtype), b, hq, hkv, nq, nk, d,
                C.bhn_strides(q_int8, tensor_layout), C.bhn_strides(k_int8, tensor_layout),
                C.bhn_strides(v_fp16, tensor_layout), C.bhn_strides(output, tensor_layout),
                1 if is_causal else 0, float(sm_scale), blk_q, blk_k, warp_q, warp_k, gran,
                _PV_CODE[pv_accum_dtype], C.stream_ptr(dev)))
    _after_launch(dev, status)
    return lse


def _sageattn_one_call(q, k, v, tensor_layout, is_causal, pv_accum_dtype, smooth_k, return_lse, qk_config,
                       sm_scale, qk_quant_gran, head_dim):
    """The path of _sageattn_configured through the single C entry point sage_b200_sageattn: one
    workspace allocation and one foreign call instead of five.  Inputs are already padded and aligned."""
    blk_q, blk_k, warp_q, warp_k = qk_config
    if qk_quant_gran == "per_warp":
        blk_q, warp_k, qk_quant_gran = warp_q, blk_k, "per_block"
    gran = C.GRAN_PER_THREAD if qk_quant_gran == "per_thread" else C.GRAN_PER_BLOCK
    b, hq, nq, d = C.bhnd(q, tensor_layout)
    _, hkv, nk, _ = C.bhnd(k, tensor_layout)
    dev = q.device
    L = C.lib()
    dt = C.dtype_code(q.dtype)
    cast_v = 0 if v.dtype == torch.float16 else 1
    nbytes = L.sage_b200_sageattn_workspace_bytes(dt, b, hq, hkv, nq, nk, d, blk_q, blk_k, warp_q, warp_k, gran,
                                                  1 if smooth_k else 0, cast_v)
    work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    output = _new_output(q, head_dim)
    lse = torch.empty((b, hq, nq), dtype=torch.float32, device=dev) if return_lse else None
    km = None
    if return_lse and smooth_k:
        km = torch.empty((b, hkv, 1, d) if tensor_layout == "HND" else (b, 1, hkv, d), dtype=k.dtype, device=dev)
    status = _launch_status(dev)
    with torch.cuda.device(dev):
        C.check(L.sage_b200_sageattn(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), output.data_ptr(), lse.data_ptr() if return_lse else 0,
            km.data_ptr() if km is not None else 0, work.data_ptr(), nbytes, status.data_ptr(),
            dt, b, hq, hkv, nq, nk, d, C.bhn_strides(q, tensor_layout), C.bhn_strides(k, tensor_layout),
            C.bhn_strides(v, tensor_layout), C.bhn_strides(output, tensor_layout), 1 if is_causal else 0,
            float(sm_scale), blk_q, blk_k, warp_q, warp_k, gran, 1 if smooth_k else 0, _PV_CODE[pv_accum_dtype],
            Q._DIV[Q.default_div_mode()], C.stream_ptr(dev)))
    _after_launch(dev, status)
    output = output[..., :head_dim]
    if not return_lse:
        return output
    lse = lse / LOG2_E
    if smooth_k:
        lse = lse + _lse_correction(q, km, tensor_layout) * sm_scale
    return output, lse


def _sageattn_traceable(q, k, v, tensor_layout, is_causal, pv_accum_dtype, smooth_k, smooth_v, return_lse, qk_config,
                        sm_scale, qk_quant_gran, head_dim):
    """The same path written with torch operators only (the natively registered ones of
    sageattention/ops.py plus torch functions), which is what torch.compile traces.  Inputs are already
    padded and aligned."""
    from .ops import ops
    blk_q, blk_k, warp_q, warp_k = qk_config
    if qk_quant_gran == "per_warp":
        blk_q, warp_k, qk_quant_gran = warp_q, blk_k, "per_block"
    per_thread = qk_quant_gran == "per_thread"
    layout = 1 if tensor_layout == "HND" else 0
    div = Q._DIV[Q.default_div_mode()]
    km = None
    if not smooth_v and pv_accum_dtype in _PV_CODE:
        output, lse, km = ops.sageattn(q, k, v, layout, is_causal, float(sm_scale), blk_q, blk_k, warp_q, warp_k,
                                       C.GRAN_PER_THREAD if per_thread else C.GRAN_PER_BLOCK, smooth_k,
                                       _PV_CODE[pv_accum_dtype], div, return_lse)
    else:
        q8, qs = ops.quant_int8(q, None, layout, blk_q, warp_q if per_thread else blk_q,
                                C.GROUP_Q_THREAD if per_thread else C.GROUP_BLOCK, div)
        km = ops.mean_k(k, layout) if smooth_k else None
        k8, ks = ops.quant_int8(k, km, layout, blk_k, warp_k if per_thread else blk_k,
                                C.GROUP_K_THREAD if per_thread else C.GROUP_BLOCK, div)
        output = torch.empty(q.size(), dtype=q.dtype, device=q.device)
        if not per_thread:
            raise ValueError("under torch.compile the fp8 and smooth_v variants take qk_quant_gran='per_thread'.")
        if pv_accum_dtype == _FP8_PV:
            v8, vs = ops.quant_v_fp8(v, layout)
            lse = ops.qk_int8_sv_f8_accum_f32_attn(q8, k8, v8, output, qs, ks, vs, layout, is_causal, float(sm_scale),
                                                   blk_q, blk_k, warp_q, warp_k, return_lse)
        else:                                                 # smooth_v with the fp16 accumulator
            seq = 2 if tensor_layout == "HND" else 1
            vm = ops.mean_k(v, layout)
            v_s = (v - vm).to(torch.float16)
            lse = ops.qk_int8_sv_f16_accum_f16_fuse_v_mean_attn(q8, k8, v_s, output, qs, ks, vm.squeeze(seq).contiguous(),
                                                                layout, is_causal, float(sm_scale), blk_q, blk_k,
                                                                warp_q, warp_k, return_lse)
    output = output[..., :head_dim]
    if not return_lse:
        return output
    lse = lse / LOG2_E
    if smooth_k:
        lse = lse + _lse_correction(q, km, tensor_layout) * sm_scale
    return output, lse


def _sageattn_configured(q, k, v, tensor_layout, is_causal, pv_accum_dtype, smooth_k, smooth_v, return_lse,
                         qk_config, sm_scale: Optional[float] = None, qk_quant_gran: str = "per_thread"):
    """Same contract as the reference's _sageattn_configured (cuda_attn.py:126-274)."""
    dtype = q.dtype
    if not q.is_cuda:
        raise ValueError("Input tensors must be CUDA tensors.")
    if dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported dtype: {dtype}")
    if q.device != k.device or q.device != v.device:
        raise ValueError("All tensors must be on the same device.")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("All tensors must have the same dtype.")
    if k.shape != v.shape:
        raise ValueError("k and v must have the same shape.")
    if tensor_layout not in ("NHD", "HND"):
        raise ValueError("tensor_layout must be 'NHD' or 'HND'.")
    if pv_accum_dtype not in _PV_CODE and pv_accum_dtype != _FP8_PV:
        raise ValueError("pv_accum_dtype must be 'fp32', 'fp16', or 'fp16+fp32'.")
    if qk_quant_gran not in ("per_thread", "per_block", "per_warp"):
        raise ValueError("qk_quant_gran must be 'per_thread', 'per_block' or 'per_warp'.")

    head_dim, q, k, v = _pad_qkv(q, k, v)
    if q.stride(-1) != 1 or k.stride(-1) != 1 or v.stride(-1) != 1:
        raise ValueError("Last dimension of q, k, and v must be contiguous.")
    if sm_scale is None:
        sm_scale = head_dim ** -0.5

    if smooth_v:
        if pv_accum_dtype in ("fp32", "fp16+fp32"):
            warnings.warn("pv_accum_dtype is fp32 or fp16+fp32, smooth_v will be ignored.", stacklevel=2)
            smooth_v = False
        elif pv_accum_dtype == _FP8_PV:
            raise ValueError("smooth_v goes with pv_accum_dtype='fp16' only.")

    blk_q, blk_k, warp_q, warp_k = qk_config
    if torch.compiler.is_compiling():
        # (the operators make their own aligned copies where a tensor needs one)
        return _sageattn_traceable(q, k, v, tensor_layout, is_causal, pv_accum_dtype, smooth_k, smooth_v, return_lse,
                                   qk_config, sm_scale, qk_quant_gran, head_dim)
    # TMA and the vector kernels need 16-byte aligned rows
    def _aligned(t):
        return t if (t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3])) else t.contiguous()
    q, k, v = _aligned(q), _aligned(k), _aligned(v)
    if _profile is None and not smooth_v and pv_accum_dtype in _PV_CODE:
        return _sageattn_one_call(q, k, v, tensor_layout, is_causal, pv_accum_dtype, smooth_k, return_lse,
                                  qk_config, sm_scale, qk_quant_gran, head_dim)
    if qk_quant_gran == "per_warp":
        # one scale per WARPQ query rows and per BLKK keys: the per-block scheme with WARPQ-row Q blocks
        blk_q, qk_config, qk_quant_gran = warp_q, (warp_q, blk_k, warp_q, blk_k), "per_block"
    per_thread = qk_quant_gran == "per_thread"
    with _Timed("quant_q"):
        q_int8, q_scale = Q._quant_one(q, None, blk_q, warp_q if per_thread else blk_q,
                                       C.GROUP_Q_THREAD if per_thread else C.GROUP_BLOCK, tensor_layout,
                                       Q.default_div_mode())
    with _Timed("smooth_quant_k"):
        k_kind = C.GROUP_K_THREAD if per_thread else C.GROUP_BLOCK
        k_warp = warp_k if per_thread else blk_k
        if smooth_k:
            km, k_int8, k_scale = Q.smooth_quant_k(k, blk_k, k_warp, k_kind, tensor_layout)
        else:
            km = None
            k_int8, k_scale = Q._quant_one(k, None, blk_k, k_warp, k_kind, tensor_layout, Q.default_div_mode())
    v_scale = None
    v_mean = None
    with _Timed("cast_v"):
        if pv_accum_dtype == _FP8_PV:
            v_fp16, v_scale = Q.quant_v_fp8(v, tensor_layout)
        elif smooth_v:
            v_fp16, v_mean = Q.smooth_v_fp16(v, tensor_layout)
        else:
            v_fp16 = cast_v_fp16(v, tensor_layout)

    output = _new_output(q, head_dim)
    with _Timed("attn"):
        lse = attn_fwd_quantized(q_int8, k_int8, v_fp16, output, q_scale, k_scale, tensor_layout, is_causal,
                                 sm_scale, qk_config, pv_accum_dtype, return_lse, qk_quant_gran, v_scale, v_mean)
    output = output[..., :head_dim]
    if not return_lse:
        return output
    lse = lse / LOG2_E
    if smooth_k:
        lse = lse + _lse_correction(q, km, tensor_layout) * sm_scale
    return output, lse


def sageattn_qk_int8_pv_fp16_cuda(q, k, v, tensor_layout="HND", is_causal=False,
                                  pv_accum_dtype=DEFAULT_PV_ACCUM_DTYPE, smooth_k=True, smooth_v=False,
                                  return_lse=False, attn_mask=None, sm_scale: Optional[float] = None,
                                  qk_quant_gran: str = "per_thread"):
    """SageAttention forward: int8 Q.K^T, fp16 P.V.  Signature of the reference
    (cuda_attn.py:44-55) plus the keyword-only extras `sm_scale` and `qk_quant_gran`."""
    assert attn_mask is None
    kv_len = k.size(2) if tensor_layout == "HND" else k.size(1)
    qk_config = select_qk_config(_padded_head_dim(q.size(-1)), is_causal, pv_accum_dtype, kv_len)
    return _sageattn_configured(q, k, v, tensor_layout, is_causal, pv_accum_dtype, smooth_k, smooth_v,
                                return_lse, qk_config, sm_scale, qk_quant_gran)


def sageattn_qk_int8_pv_fp8_cuda(q, k, v, tensor_layout="HND", is_causal=False, qk_quant_gran="per_thread",
                                 sm_scale: Optional[float] = None, pv_accum_dtype="fp32", smooth_k=True,
                                 smooth_v=False, return_lse=False, attn_mask=None):
    """SageAttention forward with fp8 (e4m3) P.V: int8 Q.K^T as in sageattn_qk_int8_pv_fp16_cuda, V
    quantised to e4m3 with one scale per channel, P rounded to e4m3, fp32 accumulation.  The name is
    the one the reference exports as a placeholder (core.py:19); the argument list follows upstream
    SageAttention2's function of that name.  `pv_accum_dtype` other than "fp32" (upstream also has
    "fp32+fp32" and "fp32+fp16" two-level schemes for sm89/sm90) is accepted and runs as fp32."""
    assert attn_mask is None
    if smooth_v:
        warnings.warn("smooth_v is not built for the fp8 path and will be ignored.", stacklevel=2)
    kv_len = k.size(2) if tensor_layout == "HND" else k.size(1)
    qk_config = select_qk_config(_padded_head_dim(q.size(-1)), is_causal, "fp32", kv_len)
    return _sageattn_configured(q, k, v, tensor_layout, is_causal, _FP8_PV, smooth_k, False, return_lse, qk_config,
                                sm_scale, qk_quant_gran)


C.lib()  # fail at import time if the native library is missing

sageattn = sageattn_qk_int8_pv_fp16_cuda

# Names other libraries probe for (reference: core.py:18-21).  The Triton backend is not part of
# this package; the sm90 fp8 variant and varlen are not built.
sageattn_qk_int8_pv_fp16_triton = None
sageattn_qk_int8_pv_fp8_cuda_sm90 = None
sageattn_varlen = None
