"""Fixed tile table.

The reference times four (BLKQ, BLKK, WARPQ, WARPK) candidates per shape at run time
(sageattention/cuda_autotune.py:9-77) because its sm80 kernel's best CTA shape depends on the
GPU.  The sm_100a kernels fix their CTA shape per accumulate mode (128-row query tiles against
128-key blocks), and what the tuple still decides is which rows and keys share an int8 scale, which must be the
same in the quantiser and in the attention kernel.  The table therefore maps
(head_dim, causal, pv_accum_dtype, sequence bucket) to the scale grouping; today every entry is
the reference's first candidate and fallback, (128, 64, 32, 64), which keeps results comparable
with the reference run under that configuration.
"""
from __future__ import annotations

QK_CONFIGS = (
    (128, 64, 32, 64),
    (128, 32, 32, 32),
    (64, 64, 32, 64),
    (128, 64, 16, 64),
)
DEFAULT_QK_CONFIG = QK_CONFIGS[0]

# groupings the sm_100a attention kernels consume: BLKK = WARPK = 64 or 32, i.e. all four
SUPPORTED_QK_CONFIGS = tuple(c for c in QK_CONFIGS if c[1] == c[3] and c[1] in (32, 64))

_SEQ_BUCKETS = (1024, 4096, 16384, 65536)


def seq_bucket(n: int) -> int:
    for i, edge in enumerate(_SEQ_BUCKETS):
        if n <= edge:
            return i
    return len(_SEQ_BUCKETS)


_TABLE = {
    (d, causal, acc, bucket): DEFAULT_QK_CONFIG
    for d in (64, 128, 256)
    for causal in (False, True)
    for acc in ("fp32", "fp16", "fp16+fp32")
    for bucket in range(len(_SEQ_BUCKETS) + 1)
}


def select_qk_config(head_dim: int, is_causal: bool, pv_accum_dtype: str, kv_len: int):
    return _TABLE.get((head_dim, bool(is_causal), pv_accum_dtype, seq_bucket(kv_len)), DEFAULT_QK_CONFIG)
