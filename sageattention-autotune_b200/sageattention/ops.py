"""Torch operators of this package and their fake (meta) implementations.

The operators themselves are registered from native code (csrc/torch_ops.cpp, built into
libsage_b200_torch.so) under the namespace ``sageattention_b200``, the way the reference registers
``sageattention_qattn_sm80`` (csrc/qattn/pybind_sm80.cpp:24-98); this module loads that library
and gives every operator a fake implementation so that ``torch.compile(fullgraph=True)`` can trace
through them, as the reference does in sageattention/cuda_compile.py:9-68.  The attention
operators keep the reference's names and argument lists.
"""
from __future__ import annotations

import os

import torch

from . import _capi as C

_HERE = os.path.dirname(os.path.abspath(__file__))
_TORCH_LIB = os.path.join(_HERE, "libsage_b200_torch.so")

C.lib()                                     # libsage_b200.so first: the operator library links against it
if not os.path.exists(_TORCH_LIB):
    raise ImportError(f"{_TORCH_LIB} is missing: build it with `python sageattention-autotune_b200/build.py`")
torch.ops.load_library(_TORCH_LIB)
ops = torch.ops.sageattention_b200

NS = "sageattention_b200"
ATTN_OPS = ("qk_int8_sv_f16_accum_f32_attn", "qk_int8_sv_f16_accum_f16_attn", "qk_int8_sv_f16_accum_f16_attn_inst_buf")
ALL_OPS = ATTN_OPS + ("qk_int8_sv_f16_accum_f16_fuse_v_mean_attn", "qk_int8_sv_f8_accum_f32_attn",
                      "qk_int8_sv_f16_attn_per_block", "mean_k", "quant_int8", "cast_v_f16", "quant_v_fp8", "sageattn")


def _bhnd(t: torch.Tensor, tensor_layout: int):
    if tensor_layout == 1:
        b, h, n, d = t.shape
    else:
        b, n, h, d = t.shape
    return b, h, n, d


def _empty_lse(query: torch.Tensor, tensor_layout: int, return_lse: bool) -> torch.Tensor:
    b, h, n, _ = _bhnd(query, tensor_layout)
    return query.new_empty((b, h, n) if return_lse else (0,), dtype=torch.float32)


def _attn_fake(query, key, value, output, query_scale, key_scale, tensor_layout, is_causal, sm_scale, blk_q, blk_k,
               warp_q, warp_k, return_lse):
    return _empty_lse(query, tensor_layout, return_lse)


for _name in ATTN_OPS:
    torch.library.register_fake(f"{NS}::{_name}")(_attn_fake)


@torch.library.register_fake(f"{NS}::qk_int8_sv_f16_accum_f16_fuse_v_mean_attn")
def _(query, key, value, output, query_scale, key_scale, value_mean, tensor_layout, is_causal, sm_scale, blk_q, blk_k,
      warp_q, warp_k, return_lse):
    return _empty_lse(query, tensor_layout, return_lse)


@torch.library.register_fake(f"{NS}::qk_int8_sv_f8_accum_f32_attn")
def _(query, key, value, output, query_scale, key_scale, value_scale, tensor_layout, is_causal, sm_scale, blk_q, blk_k,
      warp_q, warp_k, return_lse):
    return _empty_lse(query, tensor_layout, return_lse)


@torch.library.register_fake(f"{NS}::qk_int8_sv_f16_attn_per_block")
def _(query, key, value, output, query_scale, key_scale, tensor_layout, is_causal, sm_scale, blk_q, blk_k, pv_accum,
      return_lse):
    return _empty_lse(query, tensor_layout, return_lse)


@torch.library.register_fake(f"{NS}::mean_k")
def _(k, tensor_layout):
    b, h, _, d = _bhnd(k, tensor_layout)
    return k.new_empty((b, h, 1, d) if tensor_layout == 1 else (b, 1, h, d))


@torch.library.register_fake(f"{NS}::quant_int8")
def _(x, mean, tensor_layout, blk, warp, group_kind, div_mode):
    b, h, n, _ = _bhnd(x, tensor_layout)
    blocks = (n + blk - 1) // blk
    groups = blocks * (blk // warp) * 8 if group_kind == 0 else blocks * (blk // warp) * 4 if group_kind == 1 else blocks
    return x.new_empty(x.shape, dtype=torch.int8), x.new_empty((b, h, groups), dtype=torch.float32)


@torch.library.register_fake(f"{NS}::cast_v_f16")
def _(v, tensor_layout):
    return v.new_empty(v.shape, dtype=torch.float16)


@torch.library.register_fake(f"{NS}::quant_v_fp8")
def _(v, tensor_layout):
    b, h, _, d = _bhnd(v, tensor_layout)
    return v.new_empty(v.shape, dtype=torch.float8_e4m3fn), v.new_empty((b, h, d), dtype=torch.float32)


@torch.library.register_fake(f"{NS}::sageattn")
def _(q, k, v, tensor_layout, is_causal, sm_scale, blk_q, blk_k, warp_q, warp_k, granularity, smooth_k, pv_accum,
      div_mode, return_lse):
    b, h, n, _ = _bhnd(q, tensor_layout)
    _, hkv, _, d = _bhnd(k, tensor_layout)
    lse = q.new_empty((b, h, n) if return_lse else (0,), dtype=torch.float32)
    if smooth_k and return_lse:
        km = k.new_empty((b, hkv, 1, d) if tensor_layout == 1 else (b, 1, hkv, d))
    else:
        km = k.new_empty((0,))
    return q.new_empty(q.shape), lse, km
