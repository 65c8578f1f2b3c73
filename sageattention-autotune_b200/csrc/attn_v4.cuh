// SageAttention core for B200 (sm_100a), kernel for the two-level "fp16+fp32" accumulate mode.
//
// Semantics of the mode (reference: compute_fp16_sv_permuted_inst_buf, csrc/qattn/attn_utils.cuh:447-518):
// each block's P.V is accumulated in fp16 starting from zero, and that partial product is then added
// into an fp32 running output.  An fp16 accumulator in tensor memory takes one column per element, so
// one 128-row query tile per CTA fills the 512 columns: three score buffers S0..S2 (block j lives in
// S[j % 3]; its P overwrites the first 64 columns) and the fp16 partial product T.  The fp32 output
// never enters tensor memory: it lives in the registers of the fold warps.  Roles:
//   warps 0-3   softmax warpgroup A: blocks 0, 2, 4, ... (thread t = query row t, all 128 keys)
//   warps 4-7   softmax warpgroup B: blocks 1, 3, 5, ...
//   warps 8-11  fold warpgroup (thread t = query row t, holds that row of O): after every block
//               O = O * alpha + float(T) * beta; final normalisation and the output store
//   warp  12    TMA producer (one lane; also stages each block's K scales), owner of the TMEM allocation
//   warp  13    MMA issuer (whole warp runs the loop, one elected lane issues)
//   warps 14-15 idle (they only give their registers away)
// With three score buffers Q.K^T of block j+3 is issued right after P.V of block j, so a softmax
// warpgroup finds its next scores waiting; the only serial chain left is P.V(j) -> fold(j) -> P.V(j+1)
// on the single T, which is shorter than a block's softmax.
// A softmax thread reads its scores twice, 64 columns at a time (pass 1: maximum, pass 2: exponentials),
// instead of holding 128 of them: that keeps it at 144 registers and leaves 184 for a fold thread.
// The two softmax warpgroups never wait for one another: each keeps its own reference exponent and row
// sum.  A reference is an INTEGER (a multiple of kRefStep) r >= the running maximum of the blocks its
// warpgroup has seen, so P = 2^(s - r) <= 1 as the fp16 partial product requires, and every factor
// between two references is an exact power of two.  Each block's reference travels to the fold warps, which keep the output's
// own reference (the largest seen so far) and apply alpha = 2^(r_O - r_new) to O and
// beta = 2^(r_block - r_new) to T; when both are 1 for a whole warp the fold is a plain add.  To keep
// that the common case a warpgroup also folds the other's reference of three blocks earlier into its
// own (the latest one that is certain to exist, so the result is reproducible bit for bit).  The two
// row sums are combined at the end.
// Because the warpgroups are out of phase, one's tensor-memory and barrier latencies hide behind the
// other's exponentials.
#pragma once

#include "attn_common.cuh"

namespace sage {
namespace v4 {

constexpr int kRefRing = 8;        // block references: read by the fold warps, and three blocks later by the other softmax warpgroup
// Granularity of the reference exponents.  Measured at N = 32768 (sustained): 18.03 ms with 2, 17.87 with
// 4, 17.79 with 8, 17.66 with 16 - but at 16 the error against the oracle grows (max-abs 2.4e-3 instead
// of 2.0e-3: small P values reach the fp16 denormal range), so the step stays where precision is untouched.
constexpr float kRefStep = 4.0f;
constexpr int kScaleRing = 8;      // K dequantisation scales staged by the producer, one slot per block
constexpr int kThreads = 512;
// setmaxnreg is a warpgroup-wide instruction: the four warps of a group must ask for the same count
constexpr int kRegsSoftmax = 152, kRegsFold = 168, kRegsIssue = 40;
static_assert(8 * kRegsSoftmax + 4 * kRegsFold + 4 * kRegsIssue <= 2048, "register file");

enum BarIdx {
  kBarQFull = 0,
  kBarKFull = 1,                          // kKStages
  kBarKEmpty = kBarKFull + kKStages,
  kBarVFull = kBarKEmpty + kKStages,      // kVStages
  kBarVEmpty = kBarVFull + kVStages,
  kBarSFull = kBarVEmpty + kVStages,      // [buffer] = 3
  kBarPFull = kBarSFull + 3,              // [buffer] = 3, 128 arrivals
  kBarTFull = kBarPFull + 3,              // P.V of a block has retired
  kBarTFree = kBarTFull + 1,              // the fold has consumed T, 128 arrivals
  kBarStats = kBarTFree + 1,              // warpgroup A published 1/sum, 128 arrivals, single phase
  kBarSum = kBarStats + 1,                // both warpgroups finished, 256 arrivals, single phase
  kBarDrain = kBarSum + 1,
  kNumBars = kBarDrain + 1
};

template <int D>
struct SmemPlan {
  static constexpr int kQBytes = kTileQ * D;                 // int8
  static constexpr int kKBytes = kBlockKV * D;               // int8
  static constexpr int kVBytes = kBlockKV * D * 2;           // fp16
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQBytes;
  static constexpr int kVOff = kKOff + kKStages * kKBytes;
  static constexpr int kRingOff = kVOff + kVStages * kVBytes;           // float [kRefRing][128]
  static constexpr int kInvOff = kRingOff + kRefRing * kTileQ * 4;      // float [128]
  static constexpr int kPubOff = kInvOff + kTileQ * 4;                  // float [2 warpgroups][128]
  static constexpr int kSumOff = kPubOff + 2 * kTileQ * 4;              // float [128]
  static constexpr int kScaleOff = kSumOff + kTileQ * 4;                // float [kScaleRing][8]
  static constexpr int kBarOff = kScaleOff + kScaleRing * 8 * 4;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;             // slack for manual 1024-byte alignment
};

// One normalised output row (this thread's, fp32 in registers) to every peer copy of the output, peer by
// peer so that one address is live at a time.
template <int D, int OUT_DTYPE>
__device__ __forceinline__ void store_row_peers(const AttnParams& p, const unsigned short* orow, const float (&o)[D],
                                                float inv) {
#pragma unroll 1
  for (int i = 0; i < p.n_peer; ++i) {
    const char* d = reinterpret_cast<const char*>(orow) + p.peer_off[i];
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 16) {
      uint32_t w[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) w[k] = pack_out<OUT_DTYPE>(o[c0 + 2 * k] * inv, o[c0 + 2 * k + 1] * inv);
      asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(d + 2 * c0), "r"(w[0]), "r"(w[1]),
                   "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                   : "memory");
    }
  }
}

__device__ __forceinline__ int k_class(int c) { return ((c >> 6) << 2) | ((c & 7) >> 1); }

// 2^k for an integer-valued k <= 0, exactly; 0 below the normal range
__device__ __forceinline__ float pow2_int(float k) {
  const int e = static_cast<int>(fmaxf(k, -127.0f)) + 127;
  return __int_as_float(e << 23);
}

// Integer maxima of one 32-column chunk of scores, per scale class (class t owns columns 2t + 8i and
// 2t + 8i + 1): three-input maxima, started from the chunk (`first`) or continued from `mx`.
__device__ __forceinline__ void chunk_max(const uint32_t (&s)[32], int (&mx)[4], bool first) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    int v[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = static_cast<int>(s[2 * t + 8 * i]);
      v[2 * i + 1] = static_cast<int>(s[2 * t + 8 * i + 1]);
    }
    int m;
    if (first) {
      m = __vimax3_s32(v[0], v[1], v[2]);
      m = __vimax3_s32(m, v[3], v[4]);
      m = __vimax3_s32(m, v[5], v[6]);
      m = max(m, v[7]);
    } else {
      m = __vimax3_s32(mx[t], v[0], v[1]);
      m = __vimax3_s32(m, v[2], v[3]);
      m = __vimax3_s32(m, v[4], v[5]);
      m = __vimax3_s32(m, v[6], v[7]);
    }
    mx[t] = m;
  }
}

// Share of 2^x evaluated with a polynomial on the FMA pipe instead of ex2.approx.  Here 0 is best
// (N = 32768 causal, sustained: 18.1 ms with 0/8, 18.4 with 1/8, 18.9 with 2/8, 19.6 with 3/8): with
// two warpgroups out of phase the special-function unit is not the limiter and the extra
// instructions only cost power.  The two-tile kernel (attn_v1.cuh) is issue-bound and keeps 3/8.
#ifndef SAGE_V4_POLY
#define SAGE_V4_POLY 0
#endif

// P = 2^(S*a - ref) for one 32-column chunk: X = float(S) + 1.5*2^23 without a conversion (|S| < 2^22), then
// p = 2^(X*a + neg) with neg = -(1.5*2^23*a + ref), two columns of one class per packed FMA.  The 32 scores
// in `s` are replaced by 16 registers of fp16 pairs; the row sums go to the two packed accumulators.
__device__ __forceinline__ void chunk_exp(uint32_t (&s)[32], const unsigned long long (&a2)[4],
                                          const unsigned long long (&neg2)[4], unsigned long long& acc0,
                                          unsigned long long& acc1) {
  constexpr int kPolyDen = 8, kPolyNum = SAGE_V4_POLY;
#pragma unroll
  for (int c = 0; c < 32; c += 4) {
    const unsigned long long e0 = ptx::fma2(ptx::pack2(__uint_as_float(s[c + 0] + kMagicI), __uint_as_float(s[c + 1] + kMagicI)),
                                            a2[(c & 7) >> 1], neg2[(c & 7) >> 1]);
    const unsigned long long e1 = ptx::fma2(ptx::pack2(__uint_as_float(s[c + 2] + kMagicI), __uint_as_float(s[c + 3] + kMagicI)),
                                            a2[((c + 2) & 7) >> 1], neg2[((c + 2) & 7) >> 1]);
    float p0, p1, p2, p3;
    if (((c >> 2) % kPolyDen) < kPolyNum) {
      ptx::exp2_pair_poly(e0, p0, p1);
      ptx::exp2_pair_poly(e1, p2, p3);
    } else {
      float x0, x1, x2, x3;
      ptx::unpack2(e0, x0, x1);
      ptx::unpack2(e1, x2, x3);
      p0 = ptx::ex2(x0), p1 = ptx::ex2(x1), p2 = ptx::ex2(x2), p3 = ptx::ex2(x3);
    }
    acc0 = ptx::add2(acc0, ptx::pack2(p0, p1));
    acc1 = ptx::add2(acc1, ptx::pack2(p2, p3));
    s[c / 2 + 0] = ptx::pack_f16x2(p0, p1);
    s[c / 2 + 1] = ptx::pack_f16x2(p2, p3);
  }
}

// The new reference of a warpgroup after a block with maximum m_blk: integer, at least this block's
// maximum, never below anything already used, and not below the other warpgroup's reference of block
// j-3.  That block's softmax finished before the scores of block j could be issued, so the value is
// always the same one: results do not depend on how the two warpgroups happen to interleave.
// (references move in steps of kRefStep: coarse enough that the two warpgroups nearly always agree
// and the fold stays a plain add, fine enough that P keeps its fp16 precision: P's largest value in
// a row is at least 2^-kRefStep)
__device__ __forceinline__ float next_reference(float ref, float m_blk, float r_other) {
  return fmaxf(fmaxf(ref, ceilf(m_blk * (1.0f / kRefStep)) * kRefStep), r_other);
}

// One block of the softmax for one query row (thread): the scores of buffer t_s (this thread's lane) become
// P in place, `ref` and `d_sum` (this warpgroup's reference exponent and row sum) are brought up to date,
// and the block's reference is published for the fold warps and the other warpgroup.  `a` are the eight
// dequantisation constants of the block, `r_other` the other warpgroup's reference of three blocks
// earlier (or -inf), `lim` the last visible column when `need_mask`.  The caller waits for the scores
// before and signals P after.
//
// The scores stay in tensor memory and are read twice, 32 columns at a time (holding all 128 would cost
// the registers the fold warps need for O): pass 1 finds the block maximum, pass 2 writes P.  In a block
// without masked columns the reads are pipelined: the load of the next chunk is in flight while the
// current one is worked on, so only the very first load of a block is waited for in full.
__device__ __forceinline__ void softmax_block(uint32_t t_s, const float (&a)[8], bool need_mask, int lim, float r_other,
                                              float& ref, float& d_sum, float* ref_ring_slot,
                                              volatile float* ref_pub_slot) {
  if (!need_mask) {
    uint32_t sa[32], sb[32];
    int mx[4];
    // ---- pass 1
    ptx::tmem_ld32<0>(t_s, sa);
    ptx::tmem_wait_ld();
    ptx::tmem_ld32<0>(t_s + 32, sb);
    chunk_max(sa, mx, true);
    ptx::tmem_wait_ld();
    ptx::tmem_ld32<0>(t_s + 64, sa);
    chunk_max(sb, mx, false);
    float m_blk = fmaxf(fmaxf(static_cast<float>(mx[0]) * a[0], static_cast<float>(mx[1]) * a[1]),
                        fmaxf(static_cast<float>(mx[2]) * a[2], static_cast<float>(mx[3]) * a[3]));
    ptx::tmem_wait_ld();
    ptx::tmem_ld32<0>(t_s + 96, sb);
    chunk_max(sa, mx, true);
    ptx::tmem_wait_ld();
    ptx::tmem_ld32<0>(t_s, sa);                          // the first chunk again, for pass 2
    chunk_max(sb, mx, false);
    m_blk = fmaxf(m_blk, fmaxf(fmaxf(static_cast<float>(mx[0]) * a[4], static_cast<float>(mx[1]) * a[5]),
                               fmaxf(static_cast<float>(mx[2]) * a[6], static_cast<float>(mx[3]) * a[7])));

    const float r_new = next_reference(ref, m_blk, r_other);
    // a row that has seen nothing visible yet keeps a finite reference so that 2^(-inf - m) = 0
    const float m_ref = (r_new == -INFINITY) ? 0.0f : r_new;
    const float shrink = (ref == r_new) ? 1.0f : pow2_int(fmaxf(ref - m_ref, -127.0f));
    ref = r_new;
    *ref_pub_slot = r_new;
    *ref_ring_slot = r_new;       // (slot reuse: the block eight before was folded, and read by the other warpgroup, long ago)

    // ---- pass 2: the P of chunk q (32 keys, 16 registers) overwrites score columns [16 q, 16 q + 16), which
    // pass 2 has consumed by then; the load in flight at that moment reads columns further up
    unsigned long long a2[4], neg2[4];
    unsigned long long acc0 = ptx::pack2(0.0f, 0.0f), acc1 = acc0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float ng = fmaf(-kMagicF, a[t], -m_ref);
      a2[t] = ptx::pack2(a[t], a[t]);
      neg2[t] = ptx::pack2(ng, ng);
    }
    ptx::tmem_wait_ld();
    ptx::tmem_ld32<0>(t_s + 32, sb);
    chunk_exp(sa, a2, neg2, acc0, acc1);
    ptx::tmem_st16<0>(t_s, sa);
    ptx::tmem_wait_ld();
    ptx::tmem_ld32<0>(t_s + 64, sa);
    chunk_exp(sb, a2, neg2, acc0, acc1);
    ptx::tmem_st16<0>(t_s + 16, sb);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float ng = fmaf(-kMagicF, a[4 + t], -m_ref);
      a2[t] = ptx::pack2(a[4 + t], a[4 + t]);
      neg2[t] = ptx::pack2(ng, ng);
    }
    ptx::tmem_wait_ld();
    ptx::tmem_ld32<0>(t_s + 96, sb);
    chunk_exp(sa, a2, neg2, acc0, acc1);
    ptx::tmem_st16<0>(t_s + 32, sa);
    ptx::tmem_wait_ld();
    chunk_exp(sb, a2, neg2, acc0, acc1);
    ptx::tmem_st16<0>(t_s + 48, sb);
    float sum0, sum1, sum2, sum3;
    ptx::unpack2(acc0, sum0, sum1);
    ptx::unpack2(acc1, sum2, sum3);
    d_sum = d_sum * shrink + ((sum0 + sum1) + (sum2 + sum3));
    return;
  }

  // ---- a block with masked columns (the diagonal of a causal launch, the ragged end of the keys): plain
  // code, 64 columns at a time
  float m_blk = -INFINITY;
#pragma unroll 1
  for (int hf = 0; hf < 2; ++hf) {
    uint32_t s[64];
    ptx::tmem_ld32<0>(t_s + hf * 64, s);
    ptx::tmem_ld32<32>(t_s + hf * 64 + 32, s);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const float at = hf ? a[4 + ((c & 7) >> 1)] : a[(c & 7) >> 1];
      const float x = static_cast<float>(static_cast<int>(s[c])) * at;
      m_blk = fmaxf(m_blk, (hf * 64 + c <= lim) ? x : -INFINITY);
    }
  }
  const float r_new = next_reference(ref, m_blk, r_other);
  const float m_ref = (r_new == -INFINITY) ? 0.0f : r_new;
  const float shrink = (ref == r_new) ? 1.0f : pow2_int(fmaxf(ref - m_ref, -127.0f));
  ref = r_new;
  *ref_pub_slot = r_new;
  *ref_ring_slot = r_new;
  float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll 1
  for (int hf = 0; hf < 2; ++hf) {
    uint32_t s[64];
    ptx::tmem_ld32<0>(t_s + hf * 64, s);
    ptx::tmem_ld32<32>(t_s + hf * 64 + 32, s);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 64; c += 2) {
      const float at = hf ? a[4 + ((c & 7) >> 1)] : a[(c & 7) >> 1];
      const float x0 = static_cast<float>(static_cast<int>(s[c + 0])) * at;
      const float x1 = static_cast<float>(static_cast<int>(s[c + 1])) * at;
      const float p0 = (hf * 64 + c <= lim) ? ptx::ex2(x0 - m_ref) : 0.0f;
      const float p1 = (hf * 64 + c + 1 <= lim) ? ptx::ex2(x1 - m_ref) : 0.0f;
      sum0 += p0;
      sum1 += p1;
      s[c / 2] = ptx::pack_f16x2(p0, p1);
    }
    ptx::tmem_st32<0>(t_s + hf * 32, s);
  }
  d_sum = d_sum * shrink + (sum0 + sum1);
}

// ---------------------------------------------------------------------------------------------------
// softmax warpgroup `wg`: blocks wg, wg + 2, ... ; thread = query row, all 128 keys of a block
// ---------------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void softmax_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                             volatile int* abort_flag, float* ref_ring, float* inv_out,
                                             volatile float* ref_pub, float* sum_xchg, const float* k_scales,
                                             int wg, int row, int n_blocks, int q_row0, int b, int h) {
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  const int q_row = q_row0 + row;
  float q_sc;
  {
    int g = (p.gran == SAGE_B200_GRAN_PER_THREAD) ? (q_row / p.warp_q) * 8 + (q_row & 7) : q_row / p.warp_q;
    if (g >= p.q_groups) g = p.q_groups - 1;
    q_sc = p.q_scale[(static_cast<int64_t>(b) * p.heads_q + h) * p.q_groups + g];
  }

  float ref = -INFINITY;       // integer-valued reference exponent of this warpgroup's P and row sum
  float d_sum = 0.0f;          // row sum over this warpgroup's blocks, relative to `ref`
  bool ok = true;

#pragma unroll 1
  for (int j = wg; j < n_blocks; j += 2) {
    const int k0 = j * kBlockKV;
    const int buf = j % 3;
    const uint32_t t_s = tmem_base + lane_base + buf * 128;
    ok = wait_bar_warp(bars + 8 * (kBarSFull + buf), (j / 3) & 1, abort_flag, 10 + wg, p.wait_cycles);
    if (!ok) break;
    ptx::tc_fence_after();
    // the eight dequantisation constants of this block, staged by the producer with the K tile
    float a[8];
    {
      const float4 lo = *reinterpret_cast<const float4*>(k_scales + (j % kScaleRing) * 8);
      const float4 hi = *reinterpret_cast<const float4*>(k_scales + (j % kScaleRing) * 8 + 4);
      const float qs = p.scale_log2 * q_sc;
      a[0] = qs * lo.x, a[1] = qs * lo.y, a[2] = qs * lo.z, a[3] = qs * lo.w;
      a[4] = qs * hi.x, a[5] = qs * hi.y, a[6] = qs * hi.z, a[7] = qs * hi.w;
    }

    const bool need_mask = (k0 + kBlockKV > p.len_kv) || (p.causal && (k0 + kBlockKV - 1 > q_row0));
    const int lim = min(p.causal ? (q_row - k0) : kBlockKV, p.len_kv - k0 - 1);   // columns <= lim are visible

    const float r_other = (j >= 3) ? ref_ring[((j - 3) % kRefRing) * kTileQ + row] : -INFINITY;
    softmax_block(t_s, a, need_mask, lim, r_other, ref, d_sum, ref_ring + (j % kRefRing) * kTileQ + row,
                  ref_pub + wg * kTileQ + row);
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
    ptx::mbar_arrive(bars + 8 * (kBarPFull + buf));       // also publishes ref_ring (release)
  }

  // combine the two warpgroups' row sums, hand 1/sum to the fold warps, write the LSE
  if (wg == 1) sum_xchg[row] = d_sum;                     // (its final reference is in ref_pub)
  ptx::mbar_arrive(bars + 8 * kBarSum);
  if (wg == 0) {
    const bool got = wait_bar_warp(bars + 8 * kBarSum, 0, abort_flag, 14, p.wait_cycles);
    const float ref_b = ref_pub[kTileQ + row];
    const float r_fin = fmaxf(ref, ref_b);                // finite: block 0 has a visible key in every row
    const float total = d_sum * pow2_int(fmaxf(ref - r_fin, -127.0f)) +
                        ((ref_b == -INFINITY) ? 0.0f : sum_xchg[row] * pow2_int(fmaxf(ref_b - r_fin, -127.0f)));
    inv_out[row] = (ok && got && n_blocks > 0) ? ptx::rcp(total) : 0.0f;
    if (ok && got && n_blocks > 0 && p.lse != nullptr && q_row < p.len_q)
      p.lse[(static_cast<int64_t>(b) * p.heads_q + h) * p.len_q + q_row] = ptx::lg2(total) + r_fin;
    ptx::mbar_arrive(bars + 8 * kBarStats);
  }
}

// One block of the fold for one query row (thread): O = O * alpha + float(T) * beta, with T read from tensor
// memory at t_src (this thread's lane) and the factors taken from the block's and the output's references.
template <int D>
__device__ __forceinline__ void fold_block(uint32_t t_src, float (&o)[D], float& r_out, float r_blk) {
  const float r_new = fmaxf(r_out, r_blk);
  // exact powers of two (the references are integers), and at most one of them differs from 1;
  // an O that holds nothing yet is multiplied by 0
  const float alpha = (r_out == r_new) ? 1.0f : pow2_int(fmaxf(r_out - r_new, -127.0f));
  const float beta = (r_blk == r_new) ? 1.0f : pow2_int(fmaxf(r_blk - r_new, -127.0f));
  r_out = r_new;
  const bool plain = !__any_sync(0xffffffffu, alpha != 1.0f || beta != 1.0f);
  if (plain) {
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t t16[32];
      ptx::tmem_ld32<0>(t_src + c0, t16);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c0 + i] = ptx::add_f32_f16lo(o[c0 + i], t16[i]);
    }
  } else {
    const uint32_t beta16 = __half_as_ushort(__float2half_rn(beta));     // exact, or 0 below 2^-24
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t t16[32];
      ptx::tmem_ld32<0>(t_src + c0, t16);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c0 + i] = ptx::fma_f32_f16lo(t16[i], beta16, o[c0 + i] * alpha);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// fold warpgroup: O = O * alpha + float(T) * beta per block, then O / sum -> global
// ---------------------------------------------------------------------------------------------------
template <int D, int OUT_DTYPE>
__device__ __forceinline__ void fold_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                          volatile int* abort_flag, const float* ref_ring, const float* inv_in,
                                          uint8_t* stage, int row, int n_blocks, int q_row0, int b, int h) {
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  const uint32_t t_src = tmem_base + lane_base + 384;
  float o[D];                  // this row of the fp32 output, relative to 2^r_out
#pragma unroll
  for (int i = 0; i < D; ++i) o[i] = 0.0f;
  float r_out = -INFINITY;     // reference exponent O is expressed against
  bool ok = true;
#pragma unroll 1
  for (int j = 0; j < n_blocks; ++j) {
    ok = wait_bar_warp(bars + 8 * kBarTFull, j & 1, abort_flag, 30, p.wait_cycles);
    if (!ok) break;
    ptx::tc_fence_after();
    const float r_blk = ref_ring[(j % kRefRing) * kTileQ + row];
    fold_block<D>(t_src, o, r_out, r_blk);
    ptx::tc_fence_before();
    ptx::mbar_arrive(bars + 8 * kBarTFree);
  }
  if (ok) ok = wait_bar_warp(bars + 8 * kBarStats, 0, abort_flag, 40, p.wait_cycles);
  if (ok && n_blocks > 0) {
    const int q_row = q_row0 + row;
    const float inv = inv_in[row];
    if (q_row < p.len_q) {
      unsigned short* orow = static_cast<unsigned short*>(p.out) + b * p.os_b + h * p.os_h + q_row * p.os_n;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = pack_out<OUT_DTYPE>(o[c0 + 2 * i] * inv, o[c0 + 2 * i + 1] * inv);
        *reinterpret_cast<uint4*>(orow + c0) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    if (p.n_peer > 0) {
      // The same rows to every peer copy of the output.  A row per thread would leave the SM as 32-byte
      // requests, and a CTA does not retire before its requests over NVLink have been answered, so the
      // warp first lays its 32 rows out in shared memory (the first V stage: every block has been folded,
      // neither TMA nor the tensor core touches the stages any more) and then stores them with consecutive
      // lanes on consecutive 16-byte pieces: whole rows per request.
      constexpr int kPieces = D / 8;                       // 16-byte pieces of a row
      constexpr int kRowsPerStore = 32 / kPieces;
      uint8_t* mine = stage + (row & ~31) * (D * 2);       // this warp's rows
      const int lane = row & 31;
#pragma unroll
      for (int c = 0; c < kPieces; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = pack_out<OUT_DTYPE>(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
        *reinterpret_cast<uint4*>(mine + lane * (D * 2) + ((c ^ (lane % kPieces)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      __syncwarp();
      const int c = lane % kPieces;
      char* tile_out = reinterpret_cast<char*>(static_cast<unsigned short*>(p.out) + b * p.os_b + h * p.os_h) + c * 16;
#pragma unroll 1
      for (int i = 0; i < p.n_peer; ++i) {
        char* dst = tile_out + p.peer_off[i];
#pragma unroll 4
        for (int r0 = 0; r0 < 32; r0 += kRowsPerStore) {
          const int r = r0 + lane / kPieces;
          const int gq = q_row0 + (row & ~31) + r;
          if (gq < p.len_q)
            *reinterpret_cast<uint4*>(dst + gq * p.os_n * 2) =
                *reinterpret_cast<const uint4*>(mine + r * (D * 2) + ((c ^ (r % kPieces)) << 4));
        }
      }
    }
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
  float* inv_buf = reinterpret_cast<float*>(smem_gen + Plan::kInvOff);
  volatile float* ref_pub = reinterpret_cast<volatile float*>(smem_gen + Plan::kPubOff);
  float* sum_xchg = reinterpret_cast<float*>(smem_gen + Plan::kSumOff);
  float* k_scales = reinterpret_cast<float*>(smem_gen + Plan::kScaleOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int h_kv = h / (p.heads_q / p.heads_kv);
  // causal: the heaviest tiles (largest query index) go first
  const int tile_idx = p.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int q0 = tile_idx * kTileQ;

  const int kv_end = p.causal ? min(p.len_kv, q0 + kTileQ) : p.len_kv;
  const int n_blk = (kv_end + kBlockKV - 1) / kBlockKV;

  if (threadIdx.x == 0) {
    ptx::mbar_init(bars + 8 * kBarQFull, 1);
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
    ptx::mbar_init(bars + 8 * kBarSum, 2 * kTileQ);
    ptx::mbar_init(bars + 8 * kBarTFull, 1);
    ptx::mbar_init(bars + 8 * kBarTFree, kTileQ);
    ptx::mbar_init(bars + 8 * kBarStats, kTileQ);
    ptx::mbar_init(bars + 8 * kBarDrain, 1);
    // another CTA of this launch already gave up: do not queue more bounded waits behind it.  One thread
    // decides for the whole CTA, and every thread reads the verdict after the barrier below.
    *abort_flag = launch_aborted(p) ? kCodeLateCta : 0;
    ptx::fence_barrier_init();
  }
  if (threadIdx.x < 2 * kTileQ) ref_pub[threadIdx.x] = -INFINITY;
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
    softmax_role<D>(p, bars, tmem_base, abort_flag, ref_ring, inv_buf, ref_pub, sum_xchg, k_scales, warp >> 2,
                    threadIdx.x & 127, n_blk, q0, b, h);
  } else if (warp < 12) {
    ptx::reg_inc<kRegsFold>();
    fold_role<D, OUT_DTYPE>(p, bars, tmem_base, abort_flag, ref_ring, inv_buf, smem_gen + Plan::kVOff, threadIdx.x - 256, n_blk, q0, b, h);
  } else {
    ptx::reg_dec<kRegsIssue>();
    if (warp == 12 && lane == 0) {
      // ---------------- TMA producer ----------------
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      ptx::mbar_arrive_expect_tx(bars + 8 * kBarQFull, Plan::kQBytes);
      ptx::tma_load_4d(smem_base + Plan::kQOff, &tm_q, bars + 8 * kBarQFull, 0, q0, h, b);
      // K dequantisation scales of a block (eight values: four per 64-key half), loaded a block ahead
      const float* ks_base = p.k_scale + (static_cast<int64_t>(b) * p.heads_kv + h_kv) * p.k_groups;
      const bool per_thread = (p.gran == SAGE_B200_GRAN_PER_THREAD);
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
      bool ok = true;
      int j_k = 0, j_v = 0;
#pragma unroll 1
      for (int j = 0; j < n_blk && ok; ++j) {
        const int ks = j % kKStages, vs = j % kVStages;
        ok = wait_bar(bars + 8 * (kBarKEmpty + ks), ((j / kKStages) & 1) ^ 1, abort_flag, 50, p.wait_cycles);
        if (!ok) break;
        // this block's eight scales travel with the K tile: the arrive below releases the stores, and a
        // slot is reused kScaleRing blocks later, long after the softmax of this block has read it
        {
          float* dst = k_scales + (j % kScaleRing) * 8;
          *reinterpret_cast<float4*>(dst) = sc_lo;
          *reinterpret_cast<float4*>(dst + 4) = sc_hi;
          if (j + 1 < n_blk) load_scales(j + 1, sc_lo, sc_hi);
        }
        ptx::mbar_arrive_expect_tx(bars + 8 * (kBarKFull + ks), Plan::kKBytes);
        ptx::tma_load_4d(smem_base + Plan::kKOff + ks * Plan::kKBytes, &tm_k, bars + 8 * (kBarKFull + ks), 0,
                         j * kBlockKV, h_kv, b);
        j_k = j + 1;
        ok = wait_bar(bars + 8 * (kBarVEmpty + vs), ((j / kVStages) & 1) ^ 1, abort_flag, 51, p.wait_cycles);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bars + 8 * (kBarVFull + vs), Plan::kVBytes);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn)
          ptx::tma_load_4d(smem_base + Plan::kVOff + vs * Plan::kVBytes + pn * (kBlockKV * 128), &tm_v,
                           bars + 8 * (kBarVFull + vs), pn * 64, j * kBlockKV, h_kv, b);
        j_v = j + 1;
      }
      // Leave no copy in flight behind us, whatever made the roles stop: wait (bounded) for Q and for the
      // copies of the last stages' worth of blocks (earlier ones had landed before their stage was handed
      // back).  After a normal run these phases completed long ago and every wait returns at once.
      drain_bar(bars + 8 * kBarQFull, 0);
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

      // S[blk % 3] = Q . K(blk)^T
      auto issue_qk = [&](int blk) {
        const uint32_t d_t = tmem_base + (blk % 3) * 128;
        const uint64_t db0 = k_desc0 + static_cast<uint64_t>(((blk % kKStages) * Plan::kKBytes) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kStepsQK; ++s)
            ptx::mma_i8_ss(d_t, q_desc0 + static_cast<uint64_t>(s * 2), db0 + static_cast<uint64_t>(s * 2), idq, s != 0);
          ptx::tc_commit(bars + 8 * (kBarSFull + (blk % 3)));
          ptx::tc_commit(bars + 8 * (kBarKEmpty + (blk % kKStages)));
        }
        __syncwarp();
      };
      // T = P(blk) . V(blk), fp16 accumulate from zero
      auto issue_pv = [&](int blk) {
        const uint32_t d_t = tmem_base + 384;
        const uint32_t a_t = tmem_base + (blk % 3) * 128;
        const uint64_t db0 = v_desc0 + static_cast<uint64_t>(((blk % kVStages) * Plan::kVBytes) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kBlockKV / 16; ++s)
            ptx::mma_f16_ts(d_t, a_t + s * 8, db0 + static_cast<uint64_t>((s * 2048) >> 4), idp, s != 0 ? 1u : 0u);
          ptx::tc_commit(bars + 8 * kBarTFull);
          ptx::tc_commit(bars + 8 * (kBarVEmpty + (blk % kVStages)));
        }
        __syncwarp();
      };

      bool ok = wait_bar_warp(bars + 8 * kBarQFull, 0, abort_flag, 60, p.wait_cycles);
      for (int blk = 0; blk < 3 && blk < n_blk && ok; ++blk) {
        ok = wait_bar_warp(bars + 8 * (kBarKFull + blk % kKStages), 0, abort_flag, 61, p.wait_cycles);
        if (!ok) break;
        ptx::tc_fence_after();
        issue_qk(blk);
      }
#pragma unroll 1
      for (int j = 0; j < n_blk && ok; ++j) {
        ok = wait_bar_warp(bars + 8 * (kBarVFull + j % kVStages), (j / kVStages) & 1, abort_flag, 62, p.wait_cycles);
        if (!ok) break;
        ok = wait_bar_warp(bars + 8 * (kBarPFull + j % 3), (j / 3) & 1, abort_flag, 64, p.wait_cycles);
        if (!ok) break;
        ptx::tc_fence_after();
        if (j >= 1) {                                // the previous block's T has been folded
          ok = wait_bar_warp(bars + 8 * kBarTFree, (j - 1) & 1, abort_flag, 66, p.wait_cycles);
          if (!ok) break;
          ptx::tc_fence_after();
        }
        issue_pv(j);
        const int nxt = j + 3;                      // reuses the score buffer P(j) was read from
        if (nxt < n_blk) {
          ok = wait_bar_warp(bars + 8 * (kBarKFull + nxt % kKStages), (nxt / kKStages) & 1, abort_flag, 63, p.wait_cycles);
          if (!ok) break;
          issue_qk(nxt);
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
    poison_rows(p, kTileQ, q0, b, h, D);
    if (threadIdx.x == 0) publish_abort(p, *abort_flag);
  }
}

}  // namespace v4
}  // namespace sage
