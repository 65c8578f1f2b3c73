// SageAttention core for B200 (sm_100a), pipeline for the two-level "fp16+fp32" accumulate mode.
//
// Semantics of the mode (reference: compute_fp16_sv_permuted_inst_buf, csrc/qattn/attn_utils.cuh:447-518):
// each block's P.V is accumulated in fp16 starting from zero, and that partial product is then added
// into an fp32 running output.  An fp16 accumulator in tensor memory takes one column per element,
// so the partial product of a 128-key block (T, 128 columns at D = 128) cannot sit next to two score
// tiles and two outputs.  This pipeline therefore works on ONE 128-row query tile per CTA and spends
// the 512 columns on: two score buffers S0/S1 (P overwrites the first 64 columns of its buffer), T,
// and the fp32 output O.  Roles:
//   warps 0-3   softmax warpgroup, keys 0-63 of each block (thread t = query row t)
//   warps 4-7   softmax warpgroup, keys 64-127 of each block (thread t = query row t)
//   warps 8-11  fold warpgroup (thread t = query row t): O = O * alpha + float(T) after every block,
//               final normalisation and the output store
//   warp  12    TMA producer (one lane), owner of the TMEM allocation
//   warp  13    MMA issuer (whole warp runs the loop, one elected lane issues)
//   warps 14-15 idle
// 512 threads at 128 registers each; no setmaxnreg is needed because every role fits.
// Because S is double-buffered and the fold has its own warps, the softmax of block j+1, the P.V of
// block j and the fold of block j-1 overlap; the softmax warps never wait for the fold.
// Everything else (operand staging, descriptors, scale classes, bounded waits) is as in the coupled
// kernel (attn_v1.cuh).
#pragma once

#include "attn_common.cuh"

namespace sage {
namespace v3 {

constexpr int kAlphaRing = 4;      // rescale factors in flight between the softmax and the fold warps
constexpr int kThreads = 512;      // 2 softmax warpgroups, fold warpgroup, TMA/MMA warpgroup

enum BarIdx {
  kBarQFull = 0,
  kBarKFull = 1,                          // kKStages
  kBarKEmpty = kBarKFull + kKStages,
  kBarVFull = kBarKEmpty + kKStages,      // kVStages
  kBarVEmpty = kBarVFull + kVStages,
  kBarSFull = kBarVEmpty + kVStages,      // [buffer] = 2
  kBarPFull = kBarSFull + 2,              // [buffer] = 2, 128 arrivals
  kBarTFull = kBarPFull + 2,              // P.V of a block has retired
  kBarTFree = kBarTFull + 1,              // the fold has consumed T, 128 arrivals
  kBarStats = kBarTFree + 1,              // softmax published 1/sum, 128 arrivals, single phase
  kBarMax = kBarStats + 1,                // [buffer] = 2: both halves of a row wrote their block maximum, 256 arrivals
  kBarSum = kBarMax + 2,                  // both halves finished, 256 arrivals, single phase
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
  static constexpr int kAlphaOff = kVOff + kVStages * kVBytes;          // float [kAlphaRing][128]
  static constexpr int kInvOff = kAlphaOff + kAlphaRing * kTileQ * 4;   // float [128]
  static constexpr int kMaxOff = kInvOff + kTileQ * 4;                  // float [2 buffers][2 halves][128]
  static constexpr int kSumOff = kMaxOff + 4 * kTileQ * 4;              // float [128]
  static constexpr int kBarOff = kSumOff + kTileQ * 4;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;             // slack for manual 1024-byte alignment
};

__device__ __forceinline__ int k_class(int c) { return ((c >> 6) << 2) | ((c & 7) >> 1); }

// ---------------------------------------------------------------------------------------------------
// softmax warpgroups: two threads per query row, `half` 0 owns keys 0-63 of a block, `half` 1 keys
// 64-127, so that every scheduler hosts two softmax warps that hide each other's latencies.  The two
// threads of a row exchange their block maxima through shared memory and an mbarrier (bounded wait,
// unlike a named barrier) and keep partial row sums that are added at the end.
// ---------------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void softmax_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                             volatile int* abort_flag, float* alpha_ring, float* inv_out,
                                             float* max_xchg, float* sum_xchg, int half, int row, int n_blocks,
                                             int q_row0, int b, int h, int h_kv) {
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  const int q_row = q_row0 + row;
  float q_sc;
  {
    int g = (p.gran == SAGE_B200_GRAN_PER_THREAD) ? (q_row / p.warp_q) * 8 + (q_row & 7) : q_row / p.warp_q;
    if (g >= p.q_groups) g = p.q_groups - 1;
    q_sc = p.q_scale[(static_cast<int64_t>(b) * p.heads_q + h) * p.q_groups + g];
  }
  const float* ks_base = p.k_scale + (static_cast<int64_t>(b) * p.heads_kv + h_kv) * p.k_groups;
  const bool per_thread = (p.gran == SAGE_B200_GRAN_PER_THREAD);

#ifdef SAGE_TRACE
  long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long tprev = clock64();
#define V3_PH(k) do { const long long tn_ = clock64(); tacc[k] += tn_ - tprev; tprev = tn_; } while (0)
#else
#define V3_PH(k) do {} while (0)
#endif
  float m_run = -INFINITY;     // running maximum (base 2, scaled); P and O are expressed against it
  float d_sum = 0.0f;          // this thread's half of the row sum
  bool ok = true;
  // scales of one 64-key step (volatile asm keeps the load where it is written: one block ahead of its use)
  auto load_scales = [&](int step) -> float4 {
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (per_thread) {
      if (step * 4 + 3 < p.k_groups)
        asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
                     : "l"(ks_base + 4 * step));
    } else if (step < p.k_groups) {
      asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(r.x) : "l"(ks_base + step));
      r.y = r.z = r.w = r.x;
    }
    return r;
  };
  float4 ks_next = make_float4(0.f, 0.f, 0.f, 0.f);
  if (n_blocks > 0) ks_next = load_scales(half);

#pragma unroll 1
  for (int j = 0; j < n_blocks; ++j) {
    const int buf = j & 1;
    const int k0 = j * kBlockKV + half * 64;               // first key of this thread's 64 columns
    const uint32_t t_s = tmem_base + lane_base + buf * 128 + half * 64;
    // the four dequantisation constants of these 64 keys (loaded one block ahead: an L2 round trip
    // per block would otherwise stall both softmax warps of a scheduler at the same time)
    float a[4];
    {
      const float4 ks = ks_next;
      if (j + 1 < n_blocks) ks_next = load_scales(2 * (j + 1) + half);
      a[0] = p.scale_log2 * (q_sc * ks.x);
      a[1] = p.scale_log2 * (q_sc * ks.y);
      a[2] = p.scale_log2 * (q_sc * ks.z);
      a[3] = p.scale_log2 * (q_sc * ks.w);
    }

    V3_PH(0);
    ok = wait_bar_warp(bars + 8 * (kBarSFull + buf), (j >> 1) & 1, abort_flag, 10);
    if (!ok) break;
    ptx::tc_fence_after();
    V3_PH(1);

    uint32_t s[64];
    ptx::tmem_ld32<0>(t_s + 0, s);
    ptx::tmem_ld32<32>(t_s + 32, s);
    ptx::tmem_wait_ld();
    V3_PH(2);

    const bool need_mask = (k0 + 64 > p.len_kv) || (p.causal && (k0 + 63 > q_row0));
    float m_blk = -INFINITY;
    if (!need_mask) {
      // X = float(S) + 1.5*2^23 without a conversion (|S| < 2^22); X is monotonic in S, so the class
      // maxima are taken on X with three-input max and mapped back through the class's constant
#pragma unroll
      for (int c = 0; c < 64; ++c) s[c] += kMagicI;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float v[16];                                       // class t owns columns 2t + 8i, 2t + 8i + 1
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[2 * i] = __uint_as_float(s[2 * t + 8 * i]);
          v[2 * i + 1] = __uint_as_float(s[2 * t + 8 * i + 1]);
        }
        float mx = v[0];
#pragma unroll
        for (int i = 1; i < 15; i += 2) mx = ptx::max3(mx, v[i], v[i + 1]);
        mx = fmaxf(mx, v[15]);
        m_blk = fmaxf(m_blk, (mx - kMagicF) * a[t]);
      }
    } else {
      // diagonal or ragged columns: scale first, mask to -inf, keep the scaled values in place
      const int lim_causal = p.causal ? (q_row - k0) : 64;          // columns <= lim are visible
      const int lim = min(lim_causal, p.len_kv - k0 - 1);
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        float x = static_cast<float>(static_cast<int>(s[c])) * a[(c & 7) >> 1];
        x = (c <= lim) ? x : -INFINITY;
        m_blk = fmaxf(m_blk, x);
        s[c] = __float_as_uint(x);
      }
    }
    // exchange the block maximum with the thread that owns the other 64 columns of this row
    V3_PH(3);
    max_xchg[(buf * 2 + half) * kTileQ + row] = m_blk;
    ptx::mbar_arrive(bars + 8 * (kBarMax + buf));
    ok = wait_bar_warp(bars + 8 * (kBarMax + buf), (j >> 1) & 1, abort_flag, 12);
    if (!ok) break;
    m_blk = fmaxf(m_blk, max_xchg[(buf * 2 + (half ^ 1)) * kTileQ + row]);
    V3_PH(4);

    // exact running maximum: P <= 1, so the fp16 partial product cannot overflow
    const float m_new = fmaxf(m_run, m_blk);
    const float alpha = (j == 0 || m_new == m_run) ? 1.0f : ptx::ex2(m_run - m_new);
    m_run = m_new;
    // a row that has seen nothing visible yet keeps a finite reference so that 2^(-inf - m) = 0
    const float m_ref = (m_run == -INFINITY) ? 0.0f : m_run;
    // (the fold of block j-kAlphaRing has long finished: its P.V preceded Q.K^T of block j-2 in the pipe)
    if (half == 0) alpha_ring[(j % kAlphaRing) * kTileQ + row] = alpha;

    float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
    constexpr int kPolyDen = 8, kPolyNum = 3;    // share of 2^x evaluated on the FMA pipe (see attn_v1.cuh)
    if (!need_mask) {
      unsigned long long a2[4], neg2[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float ng = fmaf(-kMagicF, a[t], -m_ref);
        a2[t] = ptx::pack2(a[t], a[t]);
        neg2[t] = ptx::pack2(ng, ng);
      }
      unsigned long long acc0 = ptx::pack2(0.0f, 0.0f), acc1 = acc0;
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
        const unsigned long long e0 = ptx::fma2(ptx::pack2(__uint_as_float(s[c + 0]), __uint_as_float(s[c + 1])),
                                                a2[(c & 7) >> 1], neg2[(c & 7) >> 1]);
        const unsigned long long e1 = ptx::fma2(ptx::pack2(__uint_as_float(s[c + 2]), __uint_as_float(s[c + 3])),
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
      ptx::unpack2(acc0, sum0, sum1);
      ptx::unpack2(acc1, sum2, sum3);
    } else {
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = ptx::ex2(__uint_as_float(s[c + 0]) - m_ref);
        const float p1 = ptx::ex2(__uint_as_float(s[c + 1]) - m_ref);
        sum0 += p0;
        sum1 += p1;
        s[c / 2] = ptx::pack_f16x2(p0, p1);
      }
    }
    d_sum = d_sum * alpha + ((sum0 + sum1) + (sum2 + sum3));

    V3_PH(5);
    // P of keys [64*half, 64*half+64) of this block: 32 packed columns
    ptx::tmem_st32<0>(tmem_base + lane_base + buf * 128 + half * 32, s);
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
    ptx::mbar_arrive(bars + 8 * (kBarPFull + buf));       // also publishes alpha_ring (release)
    V3_PH(6);
  }
#ifdef SAGE_TRACE
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (row & 31) == 0)
    for (int k = 0; k < 8; ++k) p.trace[(half * 4 + (row >> 5)) * 8 + k] = tacc[k];
#endif

  // add the two halves of the row sum, hand 1/sum to the fold warps, write the LSE
  if (half == 1) sum_xchg[row] = d_sum;
  ptx::mbar_arrive(bars + 8 * kBarSum);
  if (half == 0) {
    const bool got = wait_bar_warp(bars + 8 * kBarSum, 0, abort_flag, 14);
    const float total = d_sum + sum_xchg[row];
    inv_out[row] = (ok && got && n_blocks > 0) ? ptx::rcp(total) : 0.0f;
    if (ok && got && n_blocks > 0 && p.lse != nullptr && q_row < p.len_q)
      p.lse[(static_cast<int64_t>(b) * p.heads_q + h) * p.len_q + q_row] = ptx::lg2(total) + m_run;
    ptx::mbar_arrive(bars + 8 * kBarStats);
  }
}

// ---------------------------------------------------------------------------------------------------
// fold warpgroup: O = O * alpha + float(T) per block, then O / sum -> global
// ---------------------------------------------------------------------------------------------------
template <int D, int OUT_DTYPE>
__device__ __forceinline__ void fold_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                          volatile int* abort_flag, const float* alpha_ring, const float* inv_in,
                                          int row, int n_blocks, int q_row0, int b, int h) {
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  const uint32_t t_t = tmem_base + lane_base + 256;
  const uint32_t t_o = tmem_base + lane_base + 384;
  bool ok = true;
#ifdef SAGE_TRACE
  long long facc[2] = {0, 0};
  long long fprev = clock64();
#endif
#pragma unroll 1
  for (int j = 0; j < n_blocks; ++j) {
    ok = wait_bar_warp(bars + 8 * kBarTFull, j & 1, abort_flag, 30);
    if (!ok) break;
    ptx::tc_fence_after();
#ifdef SAGE_TRACE
    { const long long tn_ = clock64(); facc[0] += tn_ - fprev; fprev = tn_; }
#endif
    const float alpha = alpha_ring[(j % kAlphaRing) * kTileQ + row];
    const bool any_rescale = __any_sync(0xffffffffu, alpha != 1.0f);
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t t16[32];
      uint32_t o[32];
      ptx::tmem_ld32<0>(t_t + c0, t16);
      if (j > 0) ptx::tmem_ld32<0>(t_o + c0, o);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float acc = (j > 0) ? __uint_as_float(o[i]) : 0.0f;
        if (any_rescale) acc *= alpha;
        o[i] = __float_as_uint(ptx::add_f32_f16lo(acc, t16[i]));
      }
      ptx::tmem_st32<0>(t_o + c0, o);
    }
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
    ptx::mbar_arrive(bars + 8 * kBarTFree);
#ifdef SAGE_TRACE
    { const long long tn_ = clock64(); facc[1] += tn_ - fprev; fprev = tn_; }
#endif
  }
#ifdef SAGE_TRACE
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && row == 0) {
    p.trace[80] = facc[0];
    p.trace[81] = facc[1];
  }
#endif
  if (ok) ok = wait_bar_warp(bars + 8 * kBarStats, 0, abort_flag, 40);
  if (ok && n_blocks > 0) {
    const int q_row = q_row0 + row;
    const float inv = inv_in[row];
    const bool store = q_row < p.len_q;
    unsigned short* orow = static_cast<unsigned short*>(p.out) + b * p.os_b + h * p.os_h + q_row * p.os_n;
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t o[32];
      ptx::tmem_ld32<0>(t_o + c0, o);
      ptx::tmem_wait_ld();
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        w[i] = pack_out<OUT_DTYPE>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
      if (store) {
#pragma unroll
        for (int i = 0; i < 16; i += 4)
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
  float* alpha_ring = reinterpret_cast<float*>(smem_gen + Plan::kAlphaOff);
  float* inv_buf = reinterpret_cast<float*>(smem_gen + Plan::kInvOff);
  float* max_xchg = reinterpret_cast<float*>(smem_gen + Plan::kMaxOff);
  float* sum_xchg = reinterpret_cast<float*>(smem_gen + Plan::kSumOff);

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
      ptx::mbar_init(bars + 8 * (kBarPFull + t), 2 * kTileQ);
      ptx::mbar_init(bars + 8 * (kBarMax + t), 2 * kTileQ);
    }
    ptx::mbar_init(bars + 8 * kBarSum, 2 * kTileQ);
    ptx::mbar_init(bars + 8 * kBarTFull, 1);
    ptx::mbar_init(bars + 8 * kBarTFree, kTileQ);
    ptx::mbar_init(bars + 8 * kBarStats, kTileQ);
    ptx::mbar_init(bars + 8 * kBarDrain, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 12) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    softmax_role<D>(p, bars, tmem_base, abort_flag, alpha_ring, inv_buf, max_xchg, sum_xchg, warp >> 2,
                    threadIdx.x & 127, n_blk, q0, b, h, h_kv);
  } else if (warp < 12) {
    fold_role<D, OUT_DTYPE>(p, bars, tmem_base, abort_flag, alpha_ring, inv_buf, threadIdx.x - 256, n_blk, q0, b, h);
  } else {
    if (warp == 12 && lane == 0) {
      // ---------------- TMA producer ----------------
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      ptx::mbar_arrive_expect_tx(bars + 8 * kBarQFull, Plan::kQBytes);
      ptx::tma_load_4d(smem_base + Plan::kQOff, &tm_q, bars + 8 * kBarQFull, 0, q0, h, b);
      bool ok = true;
#pragma unroll 1
      for (int j = 0; j < n_blk && ok; ++j) {
        const int ks = j % kKStages, vs = j % kVStages;
        ok = wait_bar(bars + 8 * (kBarKEmpty + ks), ((j / kKStages) & 1) ^ 1, abort_flag, 50);
        if (!ok) break;
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
      const uint32_t idp = idesc_pv<D, true>();               // fp16 accumulator
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
      // T = P(blk) . V(blk), fp16 accumulate from zero
      auto issue_pv = [&](int blk) {
        const uint32_t d_t = tmem_base + 256;
        const uint32_t a_t = tmem_base + (blk & 1) * 128;
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
#define V3_MPH(k) do { const long long tn_ = clock64(); macc[k] += tn_ - mprev; mprev = tn_; } while (0)
#else
#define V3_MPH(k) do {} while (0)
#endif
#pragma unroll 1
      for (int j = 0; j < n_blk && ok; ++j) {
        V3_MPH(0);
        ok = wait_bar_warp(bars + 8 * (kBarVFull + j % kVStages), (j / kVStages) & 1, abort_flag, 62);
        if (!ok) break;
        V3_MPH(1);
        ok = wait_bar_warp(bars + 8 * (kBarPFull + (j & 1)), (j >> 1) & 1, abort_flag, 64);
        if (!ok) break;
        V3_MPH(2);
        if (j > 0) {
          ok = wait_bar_warp(bars + 8 * kBarTFree, (j - 1) & 1, abort_flag, 66);     // T consumed by the fold
          if (!ok) break;
        }
        ptx::tc_fence_after();
        V3_MPH(3);
        issue_pv(j);
        V3_MPH(4);
        const int nxt = j + 2;                      // reuses the score buffer P(j) was read from
        if (nxt < n_blk) {
          ok = wait_bar_warp(bars + 8 * (kBarKFull + nxt % kKStages), (nxt / kKStages) & 1, abort_flag, 63);
          if (!ok) break;
          issue_qk(nxt);
        }
        V3_MPH(5);
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

}  // namespace v3
}  // namespace sage
