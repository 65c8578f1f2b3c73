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
//     (attn_v4.cuh, the two-level "fp16+fp32" accumulation only) as one CTA per query tile or in its
//     persistent form (attn_v5.cuh), or the two-tile kernel folding inside its softmax warps
//     ("coupled": head_dim 256 and 32-key scale blocks in that mode);
//   * how many 128-row query tiles one CTA takes: 1 for the one-tile kernel and for head_dim 256, else 2.
//     (One tile per CTA on the two-tile kernel was measured as a candidate for short sequences and
//     lost everywhere, so no entry selects it.)
// Keys: head_dim (64 / 128 / 256 after padding), causal, accumulate mode, and a bucket of the key
// length.  The measurements behind the entries are summarised in profiles/tile_table_sweep.md.
#pragma once

#include "../../include/sage_b200.h"

namespace sage {

constexpr int kSeqBucketEdges[] = {1024, 2048, 4096, 6144, 8192, 16384, 65536};
constexpr int kSeqBuckets = 8;

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
    // and its persistent form (one CTA per SM walking over the tiles) against one CTA per tile:
    //   D 128 causal  H 64:  N 1024  0.047 / 0.051   N 4096  0.336 / 0.369   N 6144  0.661 / 0.694   N 8192  1.128 / 1.115
    //                        N 16384  4.38 / 3.78    N 32768  18.9 / 15.8
    //   D  64 causal: as D 128 up to 8192 keys
    // The persistent form hides a tile's set-up and epilogue, which is what short sequences consist of;
    // it deals tiles round-robin across all heads, so once a head's K/V no longer stays in L2 next to
    // the other heads' (N = 8192 at 128 channels, later at 64) the one-CTA-per-tile form (tiles of one
    // head launched next to each other) wins.
    // Without a causal mask all tiles weigh the same and the persistent form walks plane after plane, so the
    // CTAs running together do share K/V; it then stays ahead a little longer:
    //   D 128 full  H 32 N 8192  0.934 / 0.946   H 16 N 16384  1.792 / 1.772   H 8 N 32768  3.47 / 3.40
    //   D  64 full  B 16 H 10 N 4096  1.054 / 1.159   B 4 H 10 N 8192  1.064 / 1.099   B 2 H 10 N 16384  2.087 / 2.109
    const bool persistent = is_causal ? (bucket <= 3 || (head_dim == 64 && bucket <= 4))
                                      : (bucket <= 4 || (head_dim == 64 && bucket <= 5));
    e.kernel = persistent ? SAGE_B200_KERNEL_ONE_TILE_PERSISTENT : SAGE_B200_KERNEL_ONE_TILE_FOLD;
    e.q_tiles_per_cta = 1;
  } else {
    e.kernel = (pv_accum == SAGE_B200_PV_F16_F32) ? SAGE_B200_KERNEL_TWO_TILE_COUPLED : SAGE_B200_KERNEL_TWO_TILE;
    // two-tile kernel, two query tiles per CTA against one, kernel time in ms on B200 (fp32 mode):
    //   D 128 causal H 64:  N 1024  0.044 / 0.053   N 2048  0.110 / 0.144   N 4096  0.312 / 0.447   N 16384  3.51 / 5.73
    //   D 128 full   H 64:  N 1024  0.046 / 0.067   N 2048  0.147 / 0.207   N 4096  0.460 / 0.747
    //   D  64 full B 16 H 10:  N 1024  0.098 / 0.127   N 2048  0.311 / 0.440   N 4096  1.145 / 1.602
    //   D 128 H 8 N 4096 (a launch of 128 CTAs):  causal 0.069 / 0.084   full 0.071 / 0.110
    e.q_tiles_per_cta = (head_dim == 256) ? 1 : 2;
  }
  return e;
}

}  // namespace sage
