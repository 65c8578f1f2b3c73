"""torch.library registration so that `torch.compile(fullgraph=True)` can trace through sageattn.

The reference wraps its autotuned call in a custom op with a fake implementation
(sageattention/cuda_autotune.py:80-131); here the op simply resolves the fixed tile table.
"""
from __future__ import annotations

import torch

from .tile_table import select_qk_config


@torch.library.custom_op("sageattention_b200::sageattn_fixed", mutates_args=())
def sageattn_fixed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str, is_causal: bool,
                   pv_accum_dtype: str, smooth_k: bool, smooth_v: bool, sm_scale: float,
                   qk_quant_gran: str) -> torch.Tensor:
    from .core import _padded_head_dim, _sageattn_configured
    kv_len = k.size(2) if tensor_layout == "HND" else k.size(1)
    cfg = select_qk_config(_padded_head_dim(q.size(-1)), is_causal, pv_accum_dtype, kv_len)
    out = _sageattn_configured(q, k, v, tensor_layout, is_causal, pv_accum_dtype, smooth_k, smooth_v, False,
                               cfg, None if sm_scale < 0 else sm_scale, qk_quant_gran)
    return out.contiguous() if out.size(-1) != q.size(-1) or not out.is_contiguous() else out


@sageattn_fixed.register_fake
def _(q, k, v, tensor_layout, is_causal, pv_accum_dtype, smooth_k, smooth_v, sm_scale, qk_quant_gran):
    return torch.empty_like(q)
