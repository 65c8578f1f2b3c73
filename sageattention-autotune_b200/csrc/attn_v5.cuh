// Persistent form of the one-tile kernel (attn_v4.cuh) for the two-level "fp16+fp32" accumulate mode.
//
// The one-tile kernel spends about 8 500 clocks per CTA outside its block loop: barrier and tensor-memory
// set-up, the first loads and Q.K^T before any score exists, and at the end the row sums, the
// normalisation and the store of the output tile by the fold warps while every other role is idle.
// At N = 32768 that is 3 % of a CTA's life, at N = 4096 a fifth.  Here a CTA is launched once per SM and
// walks over query tiles; its roles run as free-running pipelines over one global sequence of key blocks:
//   * the producer loads the next tile's Q (two Q slots) and keeps the K/V stage ring full across tiles;
//   * the MMA warp issues, for every block g of the sequence, P.V(g) and then Q.K^T(g + 3), whichever tile
//     g + 3 belongs to;
//   * the softmax warpgroups take a tile's blocks by parity of the LOCAL block index (so a tile's result
//     does not depend on where it falls in a CTA's sequence), reset their row state at a tile's first
//     block and publish it after its last;
//   * the fold warpgroup normalises and stores tile i while the others already work on tile i + 1.
// Set-up happens once, and a tile's epilogue hides behind the next tile's first blocks.
// Tiles are dealt to the CTAs round-robin over all heads, heaviest (causal) first, which balances a causal
// launch to about one percent without any global atomic.  The price is locality: CTAs that run together
// work on different heads, so once the K/V of all heads no longer fit L2 (N = 8192 and up for 64 heads)
// the kernel turns HBM-bound and the one-CTA-per-tile form wins; the tile table selects this form up to
// N = 4096.  (Handing tiles out from a global counter in head-major order restores the locality and was
// measured too: at N >= 16384 it is 1-2 % slower than one CTA per tile, the saved set-up being 3 % of a
// CTA's life there and the extra hand-over not free; at N = 1024 it is slower than the static deal.)  Per-tile hand-overs (row sums, references, 1/sum) go
// through eight-slot rings: the softmax can be at most four blocks ahead of the fold, every tile has at
// least one block, so a slot is never rewritten before it has been read.  At the end of a tile neither
// softmax warpgroup waits for the other: each thread publishes its row's reference and sum and bumps a
// per-row counter, and whichever of the two threads of a row comes second combines them.
//
// Arithmetic, tensor-memory plan, register split and the bounded-wait / give-up protocol are those of
// attn_v4.cuh; softmax_block and fold_block are shared with it.
#pragma once

#include "attn_v4.cuh"

namespace sage {
namespace v5 {

using v4::kRefRing;
using v4::kScaleRing;
using v4::kThreads;
using v4::kRegsSoftmax;
using v4::kRegsFold;
using v4::kRegsIssue;
constexpr int kTileRing = 8;       // per-tile hand-over slots (see the header comment)
constexpr int kQSlots = 2;

enum BarIdx {
  kBarQFull = 0,                          // kQSlots
  kBarQEmpty = kBarQFull + kQSlots,
  kBarKFull = kBarQEmpty + kQSlots,       // kKStages
  kBarKEmpty = kBarKFull + kKStages,
  kBarVFull = kBarKEmpty + kKStages,      // kVStages
  kBarVEmpty = kBarVFull + kVStages,
  kBarSFull = kBarVEmpty + kVStages,      // [buffer] = 3
  kBarPFull = kBarSFull + 3,              // [buffer] = 3, 128 arrivals
  kBarTFull = kBarPFull + 3,              // P.V of a block has retired
  kBarTFree = kBarTFull + 1,              // the fold has consumed T, 128 arrivals
  kBarStats = kBarTFree + 1,              // [kTileRing] a tile's 1/sum is published, 128 arrivals (one per row)
  kBarDrain = kBarStats + kTileRing,
  kNumBars = kBarDrain + 1
};

template <int D>
struct SmemPlan {
  static constexpr int kQBytes = kTileQ * D;                 // int8
  static constexpr int kKBytes = kBlockKV * D;               // int8
  static constexpr int kVBytes = kBlockKV * D * 2;           // fp16
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQSlots * kQBytes;
  static constexpr int kVOff = kKOff + kKStages * kKBytes;
  static constexpr int kRingOff = kVOff + kVStages * kVBytes;           // float [kRefRing][128]
  static constexpr int kInvOff = kRingOff + kRefRing * kTileQ * 4;      // float [kTileRing][128]
  static constexpr int kPubOff = kInvOff + kTileRing * kTileQ * 4;      // float [kTileRing][2][128]  a warpgroup's final reference
  static constexpr int kSumOff = kPubOff + kTileRing * 2 * kTileQ * 4;  // float [kTileRing][2][128]  a warpgroup's row sum
  static constexpr int kCntOff = kSumOff + kTileRing * 2 * kTileQ * 4;  // int   [kTileRing][128]     warpgroups that have finished the tile
  static constexpr int kScratchOff = kCntOff + kTileRing * kTileQ * 4;  // float [2][128] running references (not read by anyone else)
  static constexpr int kScaleOff = kScratchOff + 2 * kTileQ * 4;        // float [kScaleRing][8]
  static constexpr int kBarOff = kScaleOff + kScaleRing * 8 * 4;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;             // slack for manual 1024-byte alignment
};

// The tiles of this CTA, in order; CTA c takes items c, c + gridDim.x, ...  In a causal launch item i is tile
// (i / planes) of plane (i % planes), counted from the last tile down (heaviest first); otherwise it is tile
// (i % tiles) of plane (i / tiles).
struct TileWalk {
  int item, tiles, planes, total;
  int tile, h, b, q0, n_blk;
  __device__ __forceinline__ void init(const AttnParams& p) {
    tiles = (p.len_q + kTileQ - 1) / kTileQ;
    planes = p.heads_q * p.batch;
    total = tiles * planes;
    item = blockIdx.x;
    load(p);
  }
  __device__ __forceinline__ bool valid() const { return item < total; }
  __device__ __forceinline__ void load(const AttnParams& p) {
    if (item >= total) return;
    int rank, plane;
    if (p.causal) {            // all planes' heaviest tiles first: balances the CTAs without atomics
      rank = item / planes, plane = item - rank * planes;
    } else {                   // equal tiles: plane after plane, so that the CTAs running together share K/V in L2
      plane = item / tiles, rank = item - plane * tiles;
    }
    tile = p.causal ? (tiles - 1 - rank) : rank;
    h = plane % p.heads_q;
    b = plane / p.heads_q;
    q0 = tile * kTileQ;
    const int kv_end = p.causal ? min(p.len_kv, q0 + kTileQ) : p.len_kv;
    n_blk = (kv_end + kBlockKV - 1) / kBlockKV;
  }
  __device__ __forceinline__ void next(const AttnParams& p) {
    item += gridDim.x;
    load(p);
  }
};

// ---------------------------------------------------------------------------------------------------
// softmax warpgroup `wg`: of every tile the blocks wg, wg + 2, ... (local index)
// ---------------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void softmax_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                             volatile int* abort_flag, float* ref_ring, float* inv_ring,
                                             volatile float* pub_ring, volatile float* sum_ring, int* cnt_ring,
                                             volatile float* scratch, const float* k_scales, int wg, int row) {
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  TileWalk w;
  w.init(p);
  auto q_scale_of = [&](const TileWalk& t) {
    const int q_row = t.q0 + row;
    int g = (p.gran == SAGE_B200_GRAN_PER_THREAD) ? (q_row / p.warp_q) * 8 + (q_row & 7) : q_row / p.warp_q;
    if (g >= p.q_groups) g = p.q_groups - 1;
    return p.q_scale[(static_cast<int64_t>(t.b) * p.heads_q + t.h) * p.q_groups + g];
  };
  float q_sc_next = w.valid() ? q_scale_of(w) : 0.0f;
  int g0 = 0;                  // global index of the tile's first block
  bool ok = true;
#pragma unroll 1
  for (int it = 0; w.valid() && ok; ++it) {
    const float q_sc = q_sc_next;
    const int q_row0 = w.q0, q_row = w.q0 + row, n_blocks = w.n_blk;
    const int b = w.b, h = w.h;
    {                          // the next tile's query scale is fetched a tile ahead
      TileWalk nx = w;
      nx.next(p);
      if (nx.valid()) q_sc_next = q_scale_of(nx);
    }
    float ref = -INFINITY;     // integer-valued reference exponent of this warpgroup's P and row sum
    float d_sum = 0.0f;        // row sum over this warpgroup's blocks of the tile, relative to `ref`
#pragma unroll 1
    for (int j = wg; j < n_blocks; j += 2) {
      const int g = g0 + j;
      const int k0 = j * kBlockKV;
      const int buf = g % 3;
      const uint32_t t_s = tmem_base + lane_base + buf * 128;
      ok = wait_bar_warp(bars + 8 * (kBarSFull + buf), (g / 3) & 1, abort_flag, 10 + wg, p.wait_cycles);
      if (!ok) break;
      ptx::tc_fence_after();
      float a[8];
      {
        const float4 lo = *reinterpret_cast<const float4*>(k_scales + (g % kScaleRing) * 8);
        const float4 hi = *reinterpret_cast<const float4*>(k_scales + (g % kScaleRing) * 8 + 4);
        const float qs = p.scale_log2 * q_sc;
        a[0] = qs * lo.x, a[1] = qs * lo.y, a[2] = qs * lo.z, a[3] = qs * lo.w;
        a[4] = qs * hi.x, a[5] = qs * hi.y, a[6] = qs * hi.z, a[7] = qs * hi.w;
      }
      const bool need_mask = (k0 + kBlockKV > p.len_kv) || (p.causal && (k0 + kBlockKV - 1 > q_row0));
      const int lim = min(p.causal ? (q_row - k0) : kBlockKV, p.len_kv - k0 - 1);
      const float r_other = (j >= 3) ? ref_ring[((g - 3) % kRefRing) * kTileQ + row] : -INFINITY;
      v4::softmax_block(t_s, a, need_mask, lim, r_other, ref, d_sum, ref_ring + (g % kRefRing) * kTileQ + row,
                        scratch + wg * kTileQ + row);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bars + 8 * (kBarPFull + buf));     // also publishes ref_ring (release)
    }
    if (!ok) break;
    // end of the tile for this warpgroup: publish the row's reference and sum; the second of the row's two
    // threads to get here combines them, hands 1/sum to the fold warps and writes the LSE
    const int slot = it % kTileRing;
    pub_ring[(slot * 2 + wg) * kTileQ + row] = ref;
    sum_ring[(slot * 2 + wg) * kTileQ + row] = d_sum;
    __threadfence_block();
    if (atomicAdd(&cnt_ring[slot * kTileQ + row], 1) == 1) {
      __threadfence_block();
      cnt_ring[slot * kTileQ + row] = 0;                  // (the slot's next use is eight tiles away)
      const float ref_a = pub_ring[(slot * 2 + 0) * kTileQ + row], ref_b = pub_ring[(slot * 2 + 1) * kTileQ + row];
      const float sum_a = sum_ring[(slot * 2 + 0) * kTileQ + row], sum_b = sum_ring[(slot * 2 + 1) * kTileQ + row];
      const float r_fin = fmaxf(ref_a, ref_b);            // finite: block 0 has a visible key in every row
      const float total = ((ref_a == -INFINITY) ? 0.0f : sum_a * v4::pow2_int(fmaxf(ref_a - r_fin, -127.0f))) +
                          ((ref_b == -INFINITY) ? 0.0f : sum_b * v4::pow2_int(fmaxf(ref_b - r_fin, -127.0f)));
      inv_ring[slot * kTileQ + row] = ptx::rcp(total);
      if (p.lse != nullptr && q_row < p.len_q)
        p.lse[(static_cast<int64_t>(b) * p.heads_q + h) * p.len_q + q_row] = ptx::lg2(total) + r_fin;
      ptx::mbar_arrive(bars + 8 * (kBarStats + slot));    // (release: publishes inv_ring)
    }
    g0 += n_blocks;
    w.next(p);
  }
}

// ---------------------------------------------------------------------------------------------------
// fold warpgroup: O = O * alpha + float(T) * beta per block; after a tile's last block O / sum -> global
// ---------------------------------------------------------------------------------------------------
template <int D, int OUT_DTYPE>
__device__ __forceinline__ void fold_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                          volatile int* abort_flag, const float* ref_ring, const float* inv_ring,
                                          int row) {
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  const uint32_t t_src = tmem_base + lane_base + 384;
  TileWalk w;
  w.init(p);
  int g = 0;
  bool ok = true;
#pragma unroll 1
  for (int it = 0; w.valid() && ok; ++it) {
    float o[D];                // this row of the fp32 output, relative to 2^r_out
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.0f;
    float r_out = -INFINITY;   // reference exponent O is expressed against
#pragma unroll 1
    for (int j = 0; j < w.n_blk; ++j, ++g) {
      ok = wait_bar_warp(bars + 8 * kBarTFull, g & 1, abort_flag, 30, p.wait_cycles);
      if (!ok) break;
      ptx::tc_fence_after();
      const float r_blk = ref_ring[(g % kRefRing) * kTileQ + row];
      v4::fold_block<D>(t_src, o, r_out, r_blk);
      ptx::tc_fence_before();
      ptx::mbar_arrive(bars + 8 * kBarTFree);
    }
    if (!ok) break;
    const int slot = it % kTileRing;
    ok = wait_bar_warp(bars + 8 * (kBarStats + slot), (it / kTileRing) & 1, abort_flag, 40, p.wait_cycles);
    if (!ok) break;
    const int q_row = w.q0 + row;
    const float inv = inv_ring[slot * kTileQ + row];
    if (q_row < p.len_q) {
      unsigned short* orow = static_cast<unsigned short*>(p.out) + w.b * p.os_b + w.h * p.os_h + q_row * p.os_n;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 8) {
        uint32_t wd[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) wd[i] = pack_out<OUT_DTYPE>(o[c0 + 2 * i] * inv, o[c0 + 2 * i + 1] * inv);
        *reinterpret_cast<uint4*>(orow + c0) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
      }
      if (p.n_peer > 0) v4::store_row_peers<D, OUT_DTYPE>(p, orow, o, inv);
    }
    w.next(p);
  }
  ptx::tc_fence_before();
}

template <int D, int OUT_DTYPE>
__global__ void __launch_bounds__(kThreads, 1)
sage_attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using Plan = SmemPlan<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bars = smem_base + Plan::kBarOff;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + Plan::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + Plan::kMiscOff + 4);
  float* ref_ring = reinterpret_cast<float*>(smem_gen + Plan::kRingOff);
  float* inv_ring = reinterpret_cast<float*>(smem_gen + Plan::kInvOff);
  volatile float* pub_ring = reinterpret_cast<volatile float*>(smem_gen + Plan::kPubOff);
  volatile float* sum_ring = reinterpret_cast<volatile float*>(smem_gen + Plan::kSumOff);
  int* cnt_ring = reinterpret_cast<int*>(smem_gen + Plan::kCntOff);
  volatile float* scratch = reinterpret_cast<volatile float*>(smem_gen + Plan::kScratchOff);
  float* k_scales = reinterpret_cast<float*>(smem_gen + Plan::kScaleOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kQSlots; ++s) {
      ptx::mbar_init(bars + 8 * (kBarQFull + s), 1);
      ptx::mbar_init(bars + 8 * (kBarQEmpty + s), 1);
    }
    for (int s = 0; s < kKStages; ++s) {
      ptx::mbar_init(bars + 8 * (kBarKFull + s), 1);
      ptx::mbar_init(bars + 8 * (kBarKEmpty + s), 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      ptx::mbar_init(bars + 8 * (kBarVFull + s), 1);
      ptx::mbar_init(bars + 8 * (kBarVEmpty + s), 1);
    }
    for (int t = 0; t < 3; ++t) {
      ptx::mbar_init(bars + 8 * (kBarSFull + t), 1);
      ptx::mbar_init(bars + 8 * (kBarPFull + t), kTileQ);
    }
    ptx::mbar_init(bars + 8 * kBarTFull, 1);
    ptx::mbar_init(bars + 8 * kBarTFree, kTileQ);
    for (int t = 0; t < kTileRing; ++t) {
      ptx::mbar_init(bars + 8 * (kBarStats + t), kTileQ);
    }
    ptx::mbar_init(bars + 8 * kBarDrain, 1);
    // another CTA of this launch already gave up: do not queue more bounded waits behind it.  One thread
    // decides for the whole CTA, and every thread reads the verdict after the barrier below.
    *abort_flag = launch_aborted(p) ? kCodeLateCta : 0;
    ptx::fence_barrier_init();
  }
  for (int i = threadIdx.x; i < kTileRing * kTileQ; i += kThreads) cnt_ring[i] = 0;
  if (warp == 12) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // the set-up above touched no global memory; what follows reads what the previous kernel wrote
  pdl_trigger();
  pdl_wait();
  const bool late = (*abort_flag != 0);

  if (late) {
    // nothing was issued: fall through to the teardown
  } else if (warp < 8) {
    ptx::reg_inc<kRegsSoftmax>();
    softmax_role<D>(p, bars, tmem_base, abort_flag, ref_ring, inv_ring, pub_ring, sum_ring, cnt_ring, scratch, k_scales, warp >> 2,
                    threadIdx.x & 127);
  } else if (warp < 12) {
    ptx::reg_inc<kRegsFold>();
    fold_role<D, OUT_DTYPE>(p, bars, tmem_base, abort_flag, ref_ring, inv_ring, threadIdx.x - 256);
  } else {
    ptx::reg_dec<kRegsIssue>();
    if (warp == 12 && lane == 0) {
      // ---------------- TMA producer ----------------
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      const bool per_thread = (p.gran == SAGE_B200_GRAN_PER_THREAD);
      TileWalk w;
      w.init(p);
      bool ok = true;
      int g = 0;               // global block index
      int q_issued = 0, j_k = 0, j_v = 0;   // tiles whose Q, blocks whose K / V copy was issued
#pragma unroll 1
      for (int it = 0; w.valid() && ok; ++it) {
        const int h_kv = w.h / (p.heads_q / p.heads_kv);
        const int qs = it % kQSlots;
        ok = wait_bar(bars + 8 * (kBarQEmpty + qs), ((it / kQSlots) & 1) ^ 1, abort_flag, 52, p.wait_cycles);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bars + 8 * (kBarQFull + qs), Plan::kQBytes);
        ptx::tma_load_4d(smem_base + Plan::kQOff + qs * Plan::kQBytes, &tm_q, bars + 8 * (kBarQFull + qs), 0, w.q0, w.h, w.b);
        q_issued = it + 1;
        // K dequantisation scales of a block (eight values: four per 64-key half)
        const float* ks_base = p.k_scale + (static_cast<int64_t>(w.b) * p.heads_kv + h_kv) * p.k_groups;
        auto load_scales = [&](int j, float4& lo, float4& hi) {
          lo = make_float4(0.f, 0.f, 0.f, 0.f);
          hi = lo;
          if (per_thread) {
            if (j * 8 + 3 < p.k_groups)
              asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(lo.x), "=f"(lo.y), "=f"(lo.z), "=f"(lo.w) : "l"(ks_base + 8 * j));
            if (j * 8 + 7 < p.k_groups)
              asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(hi.x), "=f"(hi.y), "=f"(hi.z), "=f"(hi.w) : "l"(ks_base + 8 * j + 4));
          } else {
            if (2 * j < p.k_groups) {
              asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(lo.x) : "l"(ks_base + 2 * j));
              lo.y = lo.z = lo.w = lo.x;
            }
            if (2 * j + 1 < p.k_groups) {
              asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(hi.x) : "l"(ks_base + 2 * j + 1));
              hi.y = hi.z = hi.w = hi.x;
            }
          }
        };
        float4 sc_lo, sc_hi;
        load_scales(0, sc_lo, sc_hi);
#pragma unroll 1
        for (int j = 0; j < w.n_blk && ok; ++j, ++g) {
          const int ks = g % kKStages, vs = g % kVStages;
          ok = wait_bar(bars + 8 * (kBarKEmpty + ks), ((g / kKStages) & 1) ^ 1, abort_flag, 50, p.wait_cycles);
          if (!ok) break;
          {
            float* dst = k_scales + (g % kScaleRing) * 8;
            *reinterpret_cast<float4*>(dst) = sc_lo;
            *reinterpret_cast<float4*>(dst + 4) = sc_hi;
            if (j + 1 < w.n_blk) load_scales(j + 1, sc_lo, sc_hi);
          }
          ptx::mbar_arrive_expect_tx(bars + 8 * (kBarKFull + ks), Plan::kKBytes);
          ptx::tma_load_4d(smem_base + Plan::kKOff + ks * Plan::kKBytes, &tm_k, bars + 8 * (kBarKFull + ks), 0,
                           j * kBlockKV, h_kv, w.b);
          j_k = g + 1;
          ok = wait_bar(bars + 8 * (kBarVEmpty + vs), ((g / kVStages) & 1) ^ 1, abort_flag, 51, p.wait_cycles);
          if (!ok) break;
          ptx::mbar_arrive_expect_tx(bars + 8 * (kBarVFull + vs), Plan::kVBytes);
#pragma unroll
          for (int pn = 0; pn < D / 64; ++pn)
            ptx::tma_load_4d(smem_base + Plan::kVOff + vs * Plan::kVBytes + pn * (kBlockKV * 128), &tm_v,
                             bars + 8 * (kBarVFull + vs), pn * 64, j * kBlockKV, h_kv, w.b);
          j_v = g + 1;
        }
        w.next(p);
      }
      // Leave no copy in flight behind us, whatever made the roles stop: wait (bounded) for the last Q
      // slots' and the last stages' worth of copies (earlier ones had landed before their buffer was handed
      // back).  After a normal run these phases completed long ago and every wait returns at once.
      for (int t = max(0, q_issued - kQSlots); t < q_issued; ++t)
        drain_bar(bars + 8 * (kBarQFull + t % kQSlots), (t / kQSlots) & 1);
      for (int j = max(0, j_k - kKStages); j < j_k; ++j)
        drain_bar(bars + 8 * (kBarKFull + j % kKStages), (j / kKStages) & 1);
      for (int j = max(0, j_v - kVStages); j < j_v; ++j)
        drain_bar(bars + 8 * (kBarVFull + j % kVStages), (j / kVStages) & 1);
    } else if (warp == 13) {
      // ---------------- MMA issuer ----------------
      constexpr int kRowBytesQK = (D == 64) ? 64 : 128;
      constexpr int kStepsQK = kRowBytesQK / 32;              // int8: 32 bytes of K per instruction
      const uint32_t idq = idesc_qk();
      const uint32_t idp = idesc_pv<D, true>();               // fp16 accumulator
      const uint64_t q_desc0 = desc_kmajor<kRowBytesQK>(smem_base + Plan::kQOff);
      const uint64_t k_desc0 = desc_kmajor<kRowBytesQK>(smem_base + Plan::kKOff);
      const uint64_t v_desc0 = desc_mnmajor(smem_base + Plan::kVOff, kBlockKV * 128);

      // S[g % 3] = Q(slot) . K(g)^T; `last` = this is its tile's last block: the Q slot is free afterwards
      auto issue_qk = [&](int g, int q_slot, bool last) {
        const uint32_t d_t = tmem_base + (g % 3) * 128;
        const uint64_t da0 = q_desc0 + static_cast<uint64_t>((q_slot * Plan::kQBytes) >> 4);
        const uint64_t db0 = k_desc0 + static_cast<uint64_t>(((g % kKStages) * Plan::kKBytes) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kStepsQK; ++s)
            ptx::mma_i8_ss(d_t, da0 + static_cast<uint64_t>(s * 2), db0 + static_cast<uint64_t>(s * 2), idq, s != 0);
          ptx::tc_commit(bars + 8 * (kBarSFull + (g % 3)));
          ptx::tc_commit(bars + 8 * (kBarKEmpty + (g % kKStages)));
          if (last) ptx::tc_commit(bars + 8 * (kBarQEmpty + q_slot));
        }
        __syncwarp();
      };
      // T = P(g) . V(g), fp16 accumulate from zero
      auto issue_pv = [&](int g) {
        const uint32_t d_t = tmem_base + 384;
        const uint32_t a_t = tmem_base + (g % 3) * 128;
        const uint64_t db0 = v_desc0 + static_cast<uint64_t>(((g % kVStages) * Plan::kVBytes) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kBlockKV / 16; ++s)
            ptx::mma_f16_ts(d_t, a_t + s * 8, db0 + static_cast<uint64_t>((s * 2048) >> 4), idp, s != 0 ? 1u : 0u);
          ptx::tc_commit(bars + 8 * kBarTFull);
          ptx::tc_commit(bars + 8 * (kBarVEmpty + (g % kVStages)));
        }
        __syncwarp();
      };

      // cursor of the Q.K^T issue: runs three blocks ahead of the P.V cursor
      TileWalk wq;
      wq.init(p);
      int it_q = 0, jq = 0, gq = 0;
      bool ok = true;
      // issue Q.K^T of the block under the cursor and advance it (no-op past the last tile)
      auto step_qk = [&]() {
        if (!wq.valid()) return;
        const int slot = it_q % kQSlots;
        if (jq == 0) {
          ok = wait_bar_warp(bars + 8 * (kBarQFull + slot), (it_q / kQSlots) & 1, abort_flag, 60, p.wait_cycles);
          if (!ok) return;
        }
        ok = wait_bar_warp(bars + 8 * (kBarKFull + gq % kKStages), (gq / kKStages) & 1, abort_flag, 61, p.wait_cycles);
        if (!ok) return;
        ptx::tc_fence_after();
        issue_qk(gq, slot, jq == wq.n_blk - 1);
        ++gq;
        if (++jq == wq.n_blk) {
          jq = 0;
          ++it_q;
          wq.next(p);
        }
      };
      for (int i = 0; i < 3 && ok; ++i) step_qk();

      TileWalk wp;
      wp.init(p);
      int gp = 0;
#pragma unroll 1
      for (; wp.valid() && ok; wp.next(p)) {
#pragma unroll 1
        for (int j = 0; j < wp.n_blk && ok; ++j, ++gp) {
          ok = wait_bar_warp(bars + 8 * (kBarVFull + gp % kVStages), (gp / kVStages) & 1, abort_flag, 62, p.wait_cycles);
          if (!ok) break;
          ok = wait_bar_warp(bars + 8 * (kBarPFull + gp % 3), (gp / 3) & 1, abort_flag, 64, p.wait_cycles);
          if (!ok) break;
          ptx::tc_fence_after();
          if (gp >= 1) {                               // the previous block's T has been folded
            ok = wait_bar_warp(bars + 8 * kBarTFree, (gp - 1) & 1, abort_flag, 66, p.wait_cycles);
            if (!ok) break;
            ptx::tc_fence_after();
          }
          issue_pv(gp);
          step_qk();                                   // block gp + 3 reuses the score buffer P(gp) was read from
        }
      }
      // everything this warp issued must have retired before tensor memory is released
      if (ptx::elect_one()) ptx::tc_commit(bars + 8 * kBarDrain);
      __syncwarp();
      for (int i = 0; i < (1 << 20) && !ptx::mbar_try_wait(bars + 8 * kBarDrain, 0); ++i) {}
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (warp == 12) ptx::tmem_dealloc(tmem_base, 512);
  if (*abort_flag != 0) {
    // every tile this CTA was dealt reads as NaN: which of them had been finished is not recorded
    TileWalk w;
    for (w.init(p); w.valid(); w.next(p)) poison_rows(p, kTileQ, w.q0, w.b, w.h, D);
    if (threadIdx.x == 0) publish_abort(p, *abort_flag);
  }
}

}  // namespace v5
}  // namespace sage
