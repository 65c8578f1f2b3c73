// SageAttention core for B200 (sm_100a), pipeline for the two-level "fp16+fp32" accumulate mode with
// two INDEPENDENT softmax warpgroups on one query tile.
//
// Semantics of the mode (reference: compute_fp16_sv_permuted_inst_buf, csrc/qattn/attn_utils.cuh:447-518):
// each block's P.V is accumulated in fp16 starting from zero, and that partial product is then added
// into an fp32 running output.  An fp16 accumulator in tensor memory takes one column per element, so
// one 128-row query tile per CTA uses all 512 columns: two score buffers S0/S1 (P overwrites the first
// 64 columns of its buffer), the fp16 partial product T, and the fp32 output O.  Roles:
//   warps 0-3   softmax warpgroup A: blocks 0, 2, 4, ... in S0 (thread t = query row t, all 128 keys)
//   warps 4-7   softmax warpgroup B: blocks 1, 3, 5, ... in S1
//   warps 8-11  fold warpgroup (thread t = query row t): O = O * alpha + float(T) * beta after every
//               block, final normalisation and the output store
//   warp  12    TMA producer (one lane), owner of the TMEM allocation
//   warp  13    MMA issuer (whole warp runs the loop, one elected lane issues)
//   warps 14-15 idle (they only give their registers away)
// The two softmax warpgroups never wait for one another: each keeps its own reference exponent and row
// sum.  A reference is an INTEGER r >= the running maximum of the blocks its warpgroup has seen, so
// P = 2^(s - r) <= 1 as the fp16 partial product requires, and every factor between two references
// is an exact power of two.  Each block's reference travels to the fold warps, which keep the output's
// own reference (the largest seen so far) and apply alpha = 2^(r_O - r_new) to O and
// beta = 2^(r_block - r_new) to T; when both are 1 for a whole warp the fold is a plain add.  To keep
// that the common case a warpgroup also folds the other's last published reference into its own
// (an unsynchronised read: any earlier value is equally valid).  The two row sums are combined at the end.
// Because the warpgroups are out of phase, one's tensor-memory and barrier latencies hide behind the
// other's exponentials; the variant with two threads per row (attn_v3.cuh) stalls both at once.
#pragma once

#include "attn_common.cuh"

namespace sage {
namespace v4 {

constexpr int kRefRing = 4;        // block references in flight between the softmax and the fold warps
constexpr int kScaleRing = 8;      // K dequantisation scales staged by the producer, one slot per block
constexpr int kThreads = 512;
// setmaxnreg is a warpgroup-wide instruction: the four warps of a group must ask for the same count
constexpr int kRegsSoftmax = 208, kRegsFold = 56, kRegsIssue = 40;
static_assert(8 * kRegsSoftmax + 4 * kRegsFold + 4 * kRegsIssue <= 2048, "register file");

enum BarIdx {
  kBarQFull = 0,
  kBarKFull = 1,                          // kKStages
  kBarKEmpty = kBarKFull + kKStages,
  kBarVFull = kBarKEmpty + kKStages,      // kVStages
  kBarVEmpty = kBarVFull + kVStages,
  kBarSFull = kBarVEmpty + kVStages,      // [buffer] = 2
  kBarPFull = kBarSFull + 2,              // [buffer] = 2, 128 arrivals
  kBarTFull = kBarPFull + 2,              // [slot] = 2: a 64-channel unit of P.V has retired
  kBarTFree = kBarTFull + 2,              // [slot] = 2: the fold has consumed the unit, 128 arrivals
  kBarStats = kBarTFree + 2,              // warpgroup A published 1/sum, 128 arrivals, single phase
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

__device__ __forceinline__ int k_class(int c) { return ((c >> 6) << 2) | ((c & 7) >> 1); }

// 2^k for an integer-valued k <= 0, exactly; 0 below the normal range
__device__ __forceinline__ float pow2_int(float k) {
  const int e = static_cast<int>(fmaxf(k, -127.0f)) + 127;
  return __int_as_float(e << 23);
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
  const uint32_t t_s = tmem_base + lane_base + wg * 128;
  const int q_row = q_row0 + row;
  float q_sc;
  {
    int g = (p.gran == SAGE_B200_GRAN_PER_THREAD) ? (q_row / p.warp_q) * 8 + (q_row & 7) : q_row / p.warp_q;
    if (g >= p.q_groups) g = p.q_groups - 1;
    q_sc = p.q_scale[(static_cast<int64_t>(b) * p.heads_q + h) * p.q_groups + g];
  }

#ifdef SAGE_TRACE
  long long tacc[4] = {0, 0, 0, 0};
  long long tprev = clock64();
#define V4_PH(k) do { const long long tn_ = clock64(); tacc[k] += tn_ - tprev; tprev = tn_; } while (0)
#else
#define V4_PH(k) do {} while (0)
#endif
  float ref = -INFINITY;       // integer-valued reference exponent of this warpgroup's P and row sum
  float d_sum = 0.0f;          // row sum over this warpgroup's blocks, relative to `ref`
  bool ok = true;

#pragma unroll 1
  for (int j = wg; j < n_blocks; j += 2) {
    const int k0 = j * kBlockKV;
    V4_PH(0);
    ok = wait_bar_warp(bars + 8 * (kBarSFull + wg), (j >> 1) & 1, abort_flag, 10 + wg);
    if (!ok) break;
    ptx::tc_fence_after();
    V4_PH(1);
    // the eight dequantisation constants of this block, staged by the producer with the K tile
    float a[8];
    {
      const float4 lo = *reinterpret_cast<const float4*>(k_scales + (j % kScaleRing) * 8);
      const float4 hi = *reinterpret_cast<const float4*>(k_scales + (j % kScaleRing) * 8 + 4);
      const float qs = p.scale_log2 * q_sc;
      a[0] = qs * lo.x, a[1] = qs * lo.y, a[2] = qs * lo.z, a[3] = qs * lo.w;
      a[4] = qs * hi.x, a[5] = qs * hi.y, a[6] = qs * hi.z, a[7] = qs * hi.w;
    }

    uint32_t s[128];
    ptx::tmem_ld32<0>(t_s + 0, s);
    ptx::tmem_ld32<32>(t_s + 32, s);
    ptx::tmem_ld32<64>(t_s + 64, s);
    ptx::tmem_ld32<96>(t_s + 96, s);
    ptx::tmem_wait_ld();

    const bool need_mask = (k0 + kBlockKV > p.len_kv) || (p.causal && (k0 + kBlockKV - 1 > q_row0));
    float m_blk = -INFINITY;
    if (!need_mask) {
      // X = float(S) + 1.5*2^23 without a conversion (|S| < 2^22); X is monotonic in S, so the class
      // maxima are taken on X with three-input max and mapped back through the class's constant
#pragma unroll
      for (int c = 0; c < 128; ++c) s[c] += kMagicI;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int base = (t >> 2) * 64 + (t & 3) * 2;       // the class owns columns base + 8i, base + 8i + 1
        float v[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[2 * i] = __uint_as_float(s[base + 8 * i]);
          v[2 * i + 1] = __uint_as_float(s[base + 8 * i + 1]);
        }
        float mx = v[0];
#pragma unroll
        for (int i = 1; i < 15; i += 2) mx = ptx::max3(mx, v[i], v[i + 1]);
        mx = fmaxf(mx, v[15]);
        m_blk = fmaxf(m_blk, (mx - kMagicF) * a[t]);
      }
    } else {
      // diagonal or ragged block: scale first, mask to -inf, keep the scaled values in place
      const int lim_causal = p.causal ? (q_row - k0) : kBlockKV;     // columns <= lim are visible
      const int lim = min(lim_causal, p.len_kv - k0 - 1);
#pragma unroll
      for (int c = 0; c < 128; ++c) {
        float x = static_cast<float>(static_cast<int>(s[c])) * a[k_class(c)];
        x = (c <= lim) ? x : -INFINITY;
        m_blk = fmaxf(m_blk, x);
        s[c] = __float_as_uint(x);
      }
    }

    V4_PH(2);
    // new reference: integer, at least this block's maximum, never below anything already used or
    // published by the other warpgroup (whatever value of it this read happens to see)
    const float r_new = fmaxf(fmaxf(ref, ceilf(m_blk)), ref_pub[(wg ^ 1) * kTileQ + row]);
    // a row that has seen nothing visible yet keeps a finite reference so that 2^(-inf - m) = 0
    const float m_ref = (r_new == -INFINITY) ? 0.0f : r_new;
    const float shrink = (ref == r_new) ? 1.0f : pow2_int(fmaxf(ref - m_ref, -127.0f));
    ref = r_new;
    ref_pub[wg * kTileQ + row] = r_new;
    ref_ring[(j % kRefRing) * kTileQ + row] = r_new;      // (slot reuse: block j-4 was folded before S(j) existed)

    float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
    constexpr int kPolyDen = 8, kPolyNum = 3;    // share of 2^x evaluated on the FMA pipe (see attn_v1.cuh)
    if (!need_mask) {
      unsigned long long a2[8], neg2[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float ng = fmaf(-kMagicF, a[t], -m_ref);
        a2[t] = ptx::pack2(a[t], a[t]);
        neg2[t] = ptx::pack2(ng, ng);
      }
      unsigned long long acc0 = ptx::pack2(0.0f, 0.0f), acc1 = acc0;
#pragma unroll
      for (int c = 0; c < 128; c += 4) {
        const unsigned long long e0 = ptx::fma2(ptx::pack2(__uint_as_float(s[c + 0]), __uint_as_float(s[c + 1])),
                                                a2[k_class(c)], neg2[k_class(c)]);
        const unsigned long long e1 = ptx::fma2(ptx::pack2(__uint_as_float(s[c + 2]), __uint_as_float(s[c + 3])),
                                                a2[k_class(c + 2)], neg2[k_class(c + 2)]);
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
      ptx::unpack2(acc0, sum0, sum1);
      ptx::unpack2(acc1, sum2, sum3);
    } else {
#pragma unroll
      for (int c = 0; c < 128; c += 4) {
        const float p0 = ptx::ex2(__uint_as_float(s[c + 0]) - m_ref);
        const float p1 = ptx::ex2(__uint_as_float(s[c + 1]) - m_ref);
        const float p2 = ptx::ex2(__uint_as_float(s[c + 2]) - m_ref);
        const float p3 = ptx::ex2(__uint_as_float(s[c + 3]) - m_ref);
        sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
        s[c / 2 + 0] = ptx::pack_f16x2(p0, p1);
        s[c / 2 + 1] = ptx::pack_f16x2(p2, p3);
      }
    }
    d_sum = d_sum * shrink + ((sum0 + sum1) + (sum2 + sum3));

    // P of this block: 64 packed columns at the start of the score buffer
    ptx::tmem_st32<0>(t_s + 0, s);
    ptx::tmem_st32<32>(t_s + 32, s);
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
    ptx::mbar_arrive(bars + 8 * (kBarPFull + wg));        // also publishes ref_ring (release)
    V4_PH(3);
  }
#ifdef SAGE_TRACE
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (row & 31) == 0)
    for (int k = 0; k < 4; ++k) p.trace[(wg * 4 + (row >> 5)) * 8 + k] = tacc[k];
#endif

  // combine the two warpgroups' row sums, hand 1/sum to the fold warps, write the LSE
  if (wg == 1) sum_xchg[row] = d_sum;                     // (its final reference is in ref_pub)
  ptx::mbar_arrive(bars + 8 * kBarSum);
  if (wg == 0) {
    const bool got = wait_bar_warp(bars + 8 * kBarSum, 0, abort_flag, 14);
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

// ---------------------------------------------------------------------------------------------------
// fold warpgroup: O = O * alpha + float(T) * beta per block, then O / sum -> global
// ---------------------------------------------------------------------------------------------------
template <int D, int OUT_DTYPE>
__device__ __forceinline__ void fold_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                          volatile int* abort_flag, const float* ref_ring, const float* inv_in,
                                          int row, int n_blocks, int q_row0, int b, int h) {
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  const uint32_t t_t = tmem_base + lane_base + 256;
  const uint32_t t_o = tmem_base + lane_base + 384;
  constexpr int kUnits = D / 64;          // 64-channel units per block
  float r_out = -INFINITY;     // reference exponent O is expressed against
  bool ok = true;
#ifdef SAGE_TRACE
  long long facc[3] = {0, 0, 0};
  long long fprev = clock64();
#endif
#pragma unroll 1
  for (int j = 0; j < n_blocks; ++j) {
    float alpha = 1.0f, beta = 1.0f;
    bool plain = false;
#pragma unroll 1
    for (int half = 0; half < kUnits; ++half) {
      const int u = j * kUnits + half;
      const int slot = u & 1;
      ok = wait_bar_warp(bars + 8 * (kBarTFull + slot), (u >> 1) & 1, abort_flag, 30);
      if (!ok) break;
      ptx::tc_fence_after();
#ifdef SAGE_TRACE
      { const long long tn_ = clock64(); facc[0] += tn_ - fprev; fprev = tn_; }
#endif
      if (half == 0) {
        const float r_blk = ref_ring[(j % kRefRing) * kTileQ + row];
        const float r_new = fmaxf(r_out, r_blk);
        // exact powers of two (the references are integers), and at most one of them differs from 1;
        // an O that holds nothing yet is multiplied by 0
        alpha = (r_out == r_new) ? 1.0f : pow2_int(fmaxf(r_out - r_new, -127.0f));
        beta = (r_blk == r_new) ? 1.0f : pow2_int(fmaxf(r_blk - r_new, -127.0f));
        r_out = r_new;
        plain = (j > 0) && !__any_sync(0xffffffffu, alpha != 1.0f || beta != 1.0f);
      }
      const uint32_t t_src = t_t + slot * 64;
      const uint32_t t_dst = t_o + half * 64;
      if (plain) {
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
          uint32_t t16[16], o[16];
          ptx::tmem_ld16<0>(t_src + c0, t16);
          ptx::tmem_ld16<0>(t_dst + c0, o);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(ptx::add_f32_f16lo(__uint_as_float(o[i]), t16[i]));
          ptx::tmem_st16<0>(t_dst + c0, o);
        }
      } else {
        const uint32_t beta16 = __half_as_ushort(__float2half_rn(beta));     // exact, or 0 below 2^-24
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
          uint32_t t16[16], o[16];
          ptx::tmem_ld16<0>(t_src + c0, t16);
          if (j > 0) ptx::tmem_ld16<0>(t_dst + c0, o);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float acc = (j > 0) ? __uint_as_float(o[i]) * alpha : 0.0f;
            o[i] = __float_as_uint(ptx::fma_f32_f16lo(t16[i], beta16, acc));
          }
          ptx::tmem_st16<0>(t_dst + c0, o);
        }
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bars + 8 * (kBarTFree + slot));
#ifdef SAGE_TRACE
      { const long long tn_ = clock64(); facc[1] += tn_ - fprev; fprev = tn_; facc[2] += (plain && half == 0) ? 1 : 0; }
#endif
    }
    if (!ok) break;
  }
#ifdef SAGE_TRACE
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && row == 0) {
    p.trace[80] = facc[0];
    p.trace[81] = facc[1];
    p.trace[82] = facc[2];
  }
#endif
  if (ok) ok = wait_bar_warp(bars + 8 * kBarStats, 0, abort_flag, 40);
  if (ok && n_blocks > 0) {
    const int q_row = q_row0 + row;
    const float inv = inv_in[row];
    const bool store = q_row < p.len_q;
    unsigned short* orow = static_cast<unsigned short*>(p.out) + b * p.os_b + h * p.os_h + q_row * p.os_n;
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 16) {
      uint32_t o[16];
      ptx::tmem_ld16<0>(t_o + c0, o);
      ptx::tmem_wait_ld();
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        w[i] = pack_out<OUT_DTYPE>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
      if (store) {
#pragma unroll
        for (int i = 0; i < 8; i += 4)
          *reinterpret_cast<uint4*>(orow + c0 + 2 * i) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
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

  // another CTA of this launch already gave up: do not queue more bounded waits behind it
  if (launch_aborted(p)) return;

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
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(bars + 8 * (kBarSFull + t), 1);
      ptx::mbar_init(bars + 8 * (kBarPFull + t), kTileQ);
    }
    ptx::mbar_init(bars + 8 * kBarSum, 2 * kTileQ);
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(bars + 8 * (kBarTFull + t), 1);
      ptx::mbar_init(bars + 8 * (kBarTFree + t), kTileQ);
    }
    ptx::mbar_init(bars + 8 * kBarStats, kTileQ);
    ptx::mbar_init(bars + 8 * kBarDrain, 1);
    *abort_flag = 0;
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

  if (warp < 8) {
    ptx::reg_inc<kRegsSoftmax>();
    softmax_role<D>(p, bars, tmem_base, abort_flag, ref_ring, inv_buf, ref_pub, sum_xchg, k_scales, warp >> 2,
                    threadIdx.x & 127, n_blk, q0, b, h);
  } else if (warp < 12) {
    ptx::reg_dec<kRegsFold>();
    fold_role<D, OUT_DTYPE>(p, bars, tmem_base, abort_flag, ref_ring, inv_buf, threadIdx.x - 256, n_blk, q0, b, h);
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
#pragma unroll 1
      for (int j = 0; j < n_blk && ok; ++j) {
        const int ks = j % kKStages, vs = j % kVStages;
        ok = wait_bar(bars + 8 * (kBarKEmpty + ks), ((j / kKStages) & 1) ^ 1, abort_flag, 50);
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
        ok = wait_bar(bars + 8 * (kBarVEmpty + vs), ((j / kVStages) & 1) ^ 1, abort_flag, 51);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bars + 8 * (kBarVFull + vs), Plan::kVBytes);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn)
          ptx::tma_load_4d(smem_base + Plan::kVOff + vs * Plan::kVBytes + pn * (kBlockKV * 128), &tm_v,
                           bars + 8 * (kBarVFull + vs), pn * 64, j * kBlockKV, h_kv, b);
      }
      if (!ok) {
        // leave no copy in flight behind us: wait (bounded) for what was issued
        for (int s = 0; s < kKStages; ++s)
          for (int i = 0; i < 4096 && !ptx::mbar_try_wait(bars + 8 * (kBarKFull + s), 0) &&
                          !ptx::mbar_try_wait(bars + 8 * (kBarKFull + s), 1); ++i) {}
      }
    } else if (warp == 13) {
      // ---------------- MMA issuer ----------------
      constexpr int kRowBytesQK = (D == 64) ? 64 : 128;
      constexpr int kStepsQK = kRowBytesQK / 32;              // int8: 32 bytes of K per instruction
      const uint32_t idq = idesc_qk();
      const uint32_t idp = idesc_pv<64, true>();              // fp16 accumulator, 64 channels per unit
      const uint64_t q_desc0 = desc_kmajor<kRowBytesQK>(smem_base + Plan::kQOff);
      const uint64_t k_desc0 = desc_kmajor<kRowBytesQK>(smem_base + Plan::kKOff);
      const uint64_t v_desc0 = desc_mnmajor(smem_base + Plan::kVOff, kBlockKV * 128);

      // S[blk & 1] = Q . K(blk)^T
      auto issue_qk = [&](int blk) {
        const uint32_t d_t = tmem_base + (blk & 1) * 128;
        const uint64_t db0 = k_desc0 + static_cast<uint64_t>(((blk % kKStages) * Plan::kKBytes) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kStepsQK; ++s)
            ptx::mma_i8_ss(d_t, q_desc0 + static_cast<uint64_t>(s * 2), db0 + static_cast<uint64_t>(s * 2), idq, s != 0);
          ptx::tc_commit(bars + 8 * (kBarSFull + (blk & 1)));
          ptx::tc_commit(bars + 8 * (kBarKEmpty + (blk % kKStages)));
        }
        __syncwarp();
      };
      // T[slot] = P(blk) . V(blk)[:, 64 channels of unit `half`], fp16 accumulate from zero
      constexpr int kUnits = D / 64;
      auto issue_pv_unit = [&](int blk, int half, int slot, bool last) {
        const uint32_t d_t = tmem_base + 256 + slot * 64;
        const uint32_t a_t = tmem_base + (blk & 1) * 128;
        const uint64_t db0 = v_desc0 + static_cast<uint64_t>(((blk % kVStages) * Plan::kVBytes + half * (kBlockKV * 128)) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kBlockKV / 16; ++s)
            ptx::mma_f16_ts(d_t, a_t + s * 8, db0 + static_cast<uint64_t>((s * 2048) >> 4), idp, s != 0 ? 1u : 0u);
          ptx::tc_commit(bars + 8 * (kBarTFull + slot));
          if (last) ptx::tc_commit(bars + 8 * (kBarVEmpty + (blk % kVStages)));
        }
        __syncwarp();
      };

      bool ok = wait_bar_warp(bars + 8 * kBarQFull, 0, abort_flag, 60);
      for (int blk = 0; blk < 2 && blk < n_blk && ok; ++blk) {
        ok = wait_bar_warp(bars + 8 * (kBarKFull + blk % kKStages), 0, abort_flag, 61);
        if (!ok) break;
        ptx::tc_fence_after();
        issue_qk(blk);
      }
#ifdef SAGE_TRACE
      long long macc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      long long mprev = clock64();
#define V4_MPH(k) do { const long long tn_ = clock64(); macc[k] += tn_ - mprev; mprev = tn_; } while (0)
#else
#define V4_MPH(k) do {} while (0)
#endif
#pragma unroll 1
      for (int j = 0; j < n_blk && ok; ++j) {
        V4_MPH(0);
        ok = wait_bar_warp(bars + 8 * (kBarVFull + j % kVStages), (j / kVStages) & 1, abort_flag, 62);
        if (!ok) break;
        V4_MPH(1);
        ok = wait_bar_warp(bars + 8 * (kBarPFull + (j & 1)), (j >> 1) & 1, abort_flag, 64);
        if (!ok) break;
        V4_MPH(2);
        ptx::tc_fence_after();
        V4_MPH(3);
#pragma unroll 1
        for (int half = 0; half < kUnits && ok; ++half) {
          const int u = j * kUnits + half;
          if (u >= 2) {                              // the unit that used this slot has been folded
            ok = wait_bar_warp(bars + 8 * (kBarTFree + (u & 1)), ((u >> 1) - 1) & 1, abort_flag, 66);
            if (!ok) break;
            ptx::tc_fence_after();
          }
          issue_pv_unit(j, half, u & 1, half == kUnits - 1);
        }
        if (!ok) break;
        V4_MPH(4);
        const int nxt = j + 2;                      // reuses the score buffer P(j) was read from
        if (nxt < n_blk) {
          ok = wait_bar_warp(bars + 8 * (kBarKFull + nxt % kKStages), (nxt / kKStages) & 1, abort_flag, 63);
          if (!ok) break;
          issue_qk(nxt);
        }
        V4_MPH(5);
      }
#ifdef SAGE_TRACE
      if (p.trace != nullptr && lane == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
        for (int k = 0; k < 8; ++k) p.trace[64 + k] = macc[k];
#endif
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
  if (threadIdx.x == 0 && *abort_flag != 0) publish_abort(p, *abort_flag);
}

}  // namespace v4
}  // namespace sage
