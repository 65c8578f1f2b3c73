// The fixed tile table: which kernel configuration runs a given problem.
//
// The reference picks among four (BLKQ, BLKK, WARPQ, WARPK) candidates by timing them on the first
// call of every shape (sageattention/cuda_autotune.py:9-77, autotune_utils.py:97-127), because the
// best CTA shape of its sm80 kernel depends on the GPU.  This library targets one GPU, so the choice
// is made once, from measurements on B200, and stored here.  An entry fixes
//   * the scale grouping (blk_q, blk_k, warp_q, warp_k): which query rows and keys share an int8
//     scale.  The quantisers and the attention kernel read it from the same entry, so they cannot
//     disagree.  Every entry uses the reference's first candidate and fallback (128, 64, 32, 64): the
//     sm_100a kernels consume 128 x 128 score tiles whatever the grouping, so the grouping does not
//     change their speed, and this one keeps results comparable with the reference's default;
//   * the kernel: the two-tile kernel (attn_v1.cuh), the one-tile kernel with a fold warpgroup
//     (attn_v4.cuh, the two-level "fp16+fp32" accumulation only), or the two-tile kernel folding
//     inside its softmax warps ("coupled": head_dim 256 and 32-key scale blocks in that mode);
//   * for the two-tile kernel, how many 128-row query tiles one CTA takes (2, or 1 where 256-row
//     CTAs are too few to keep 148 SMs busy).
// Keys: head_dim (64 / 128 / 256 after padding), causal, accumulate mode, and a bucket of the key
// length.  The measurements behind the entries are summarised in profiles/tile_table_sweep.md.
#pragma once

#include "../../include/sage_b200.h"

namespace sage {

constexpr int kSeqBucketEdges[] = {1024, 2048, 4096, 16384, 65536};
constexpr int kSeqBuckets = 6;

// Two-tile kernel: largest bucket that runs with one query tile per CTA (-1: none).  Separate values for
// causal and full attention: a causal launch has half the work per CTA on average.
constexpr int kOneTileMaxBucketCausal = -1;
constexpr int kOneTileMaxBucketFull = -1;

inline int seq_bucket(int len_kv) {
  for (int i = 0; i < kSeqBuckets - 1; ++i)
    if (len_kv <= kSeqBucketEdges[i]) return i;
  return kSeqBuckets - 1;
}

inline sage_b200_tile_entry tile_lookup(int head_dim, int is_causal, int pv_accum, int len_kv) {
  sage_b200_tile_entry e;
  e.blk_q = 128, e.blk_k = 64, e.warp_q = 32, e.warp_k = 64;
  const int bucket = seq_bucket(len_kv);
  e.seq_bucket = bucket;
  if (pv_accum == SAGE_B200_PV_F16_F32 && head_dim != 256) {
    // one-tile kernel against the coupled two-tile kernel, kernel time in ms on B200:
    //   D 128 causal  H 64:  N 1024  0.048 / 0.063    N 4096  0.349 / 0.507    N 32768  16.2 / 24.3
    //   D  64 full    B 16 H 10 N 4096:  1.29 / 1.49
    e.kernel = SAGE_B200_KERNEL_ONE_TILE_FOLD;
    e.q_tiles_per_cta = 1;
  } else {
    e.kernel = (pv_accum == SAGE_B200_PV_F16_F32) ? SAGE_B200_KERNEL_TWO_TILE_COUPLED : SAGE_B200_KERNEL_TWO_TILE;
    // one query tile per CTA for short sequences (entries from the sweep: see the summary file)
    const int one_tile_max = is_causal ? kOneTileMaxBucketCausal : kOneTileMaxBucketFull;
    e.q_tiles_per_cta = (head_dim == 256 || bucket <= one_tile_max) ? 1 : 2;
  }
  return e;
}

}  // namespace sage
