"""Fixed tile table.

The reference times four (BLKQ, BLKK, WARPQ, WARPK) candidates per shape at run time
(sageattention/cuda_autotune.py:9-77) because its sm80 kernel's best CTA shape depends on the
GPU.  Here the choice is made once, from measurements on B200, and lives in the native library
(csrc/tile_table.h) so that every caller - this package, the torch operators, a C program - sees
the same table: an entry names the scale grouping (which query rows and keys share an int8 scale,
the same in the quantisers and in the attention kernel), the kernel that runs the problem and, for
the two-tile kernel, how many 128-row query tiles a CTA takes.  This module is the Python view of
that table; `sage_b200_attn_fwd` consults the same entries when it launches.
"""
from __future__ import annotations

import functools

import torch

from . import _capi as C

QK_CONFIGS = (
    (128, 64, 32, 64),
    (128, 32, 32, 32),
    (64, 64, 32, 64),
    (128, 64, 16, 64),
)
DEFAULT_QK_CONFIG = QK_CONFIGS[0]

# groupings the sm_100a attention kernels consume: BLKK = WARPK = 64 or 32, i.e. all four
SUPPORTED_QK_CONFIGS = tuple(c for c in QK_CONFIGS if c[1] == c[3] and c[1] in (32, 64))

KERNEL_NAMES = {0: "two_tile", 1: "one_tile_fold", 2: "two_tile_coupled", 3: "one_tile_persistent"}
_PV = {"fp32": C.PV_F32, "fp16": C.PV_F16, "fp16+fp32": C.PV_F16_F32, "fp8": C.PV_F8}


@functools.lru_cache(maxsize=None)
def _lookup(head_dim: int, is_causal: bool, pv_code: int, kv_len: int):
    entry = C.TileEntry()
    C.check(C.lib().sage_b200_tile_lookup(head_dim, 1 if is_causal else 0, pv_code, max(1, kv_len), entry))
    return ((entry.blk_q, entry.blk_k, entry.warp_q, entry.warp_k), KERNEL_NAMES[entry.kernel],
            entry.q_tiles_per_cta, entry.seq_bucket)


def select_entry(head_dim: int, is_causal: bool, pv_accum_dtype: str, kv_len: int) -> dict:
    """The whole entry: {"qk_config", "kernel", "q_tiles_per_cta", "seq_bucket"}."""
    cfg, kernel, tiles, bucket = _lookup(head_dim, bool(is_causal), _PV.get(pv_accum_dtype, C.PV_F32), int(kv_len))
    return {"qk_config": cfg, "kernel": kernel, "q_tiles_per_cta": tiles, "seq_bucket": bucket}


@torch.compiler.assume_constant_result          # a table lookup: torch.compile folds the tuple into the graph
def select_qk_config(head_dim: int, is_causal: bool, pv_accum_dtype: str, kv_len: int):
    """(BLKQ, BLKK, WARPQ, WARPK) for the quantisers and the attention call."""
    return _lookup(head_dim, bool(is_causal), _PV.get(pv_accum_dtype, C.PV_F32), int(kv_len))[0]
