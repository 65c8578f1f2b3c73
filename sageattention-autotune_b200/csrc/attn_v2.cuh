// SageAttention core for B200 (sm_100a), decoupled pipeline: int8 Q.K^T and fp16 P.V on tcgen05
// tensor cores with accumulators in tensor memory, TMA-staged operands, online softmax in two
// softmax warpgroups that never wait for the tensor core in steady state.
//
// It replaces the reference's qk_int8_sv_f16_attn_kernel
// (csrc/qattn/qk_int8_sv_f16_kernel_sm80.cuh:61-657); the arithmetic follows the same order:
// S = int32(Q.K^T) -> scale by q_scale*k_scale*sm_scale*log2(e) -> running max in base 2 ->
// P = 2^(S*a - m) rounded to fp16 -> O += P.V -> O / sum(P), with 64-key steps like the
// reference's CTA_K = 64.
//
// One CTA = one (batch, q-head) and 256 consecutive query rows = two 128-row tiles.
//   warps 0-3   softmax warpgroup of tile 0 (thread t owns query row t: TMEM lane t)
//   warps 4-7   softmax warpgroup of tile 1
//   warp  8     TMA producer (one lane) and owner of the TMEM allocation
//   warp  9     MMA issuer (one lane)
//   warps 10-11 idle (they complete the third warpgroup so that setmaxnreg can be used)
// Tensor memory, per tile (256 of the 512 columns): two S buffers of 64 columns (int32 scores of
// 64 keys each) and 128 columns of O.  P (fp16, two keys per column) overwrites the first 32
// columns of the S buffer it was computed from.  Because S is double-buffered, Q.K^T of step i+1
// is issued while the softmax of step i is still running: the softmax warps find their next
// scores ready, and the tensor core always has the other tile's and the next step's work queued.
// K and V arrive in 128-key TMA stages shared by both tiles (two steps per stage).
//
// Scales: thread t reads its own q_scale and, per 64 keys, the four k_scales of the reference's
// per-thread grouping (key c uses entry (c%8)/2), qk_int8_sv_f16_kernel_sm80.cuh:116-126.
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises an abort flag, all roles
// leave their loops, tensor memory is released and a code is written to the caller's status word.
#pragma once

#include "attn_common.cuh"

namespace sage {
namespace v2 {

constexpr int kStepKV = 64;       // keys per softmax step / per S buffer
constexpr int kStageKV = 128;     // keys per TMA stage

enum BarIdx {
  kBarQFull = 0,
  kBarKFull = 1,                          // kKStages
  kBarKEmpty = kBarKFull + kKStages,
  kBarVFull = kBarKEmpty + kKStages,      // kVStages
  kBarVEmpty = kBarVFull + kVStages,
  kBarSFull = kBarVEmpty + kVStages,      // [tile][buffer] = 4
  kBarPFull = kBarSFull + 4,              // [tile][buffer] = 4
  kBarPvDone = kBarPFull + 4,             // [tile] = 2, one phase per step
  kBarOFinal = kBarPvDone + 2,            // [tile] = 2, completes once: the tile's last P.V has retired
  kBarTurn = kBarOFinal + 2,              // [tile][warp] = 8: whose turn it is on the special-function unit
  kBarDrain = kBarTurn + 8,
  kNumBars = kBarDrain + 1
};

template <int D>
struct SmemPlan {
  static constexpr int kQBytes = kTileQ * D;                 // int8
  static constexpr int kKBytes = kStageKV * D;               // int8
  static constexpr int kVBytes = kStageKV * D * 2;           // fp16
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + 2 * kQBytes;
  static constexpr int kVOff = kKOff + kKStages * kKBytes;
  static constexpr int kBarOff = kVOff + kVStages * kVBytes;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;             // slack for manual 1024-byte alignment
};

__host__ __device__ constexpr uint32_t idesc_qk64() {
  // int8 x int8 -> int32, both K-major, M = 128, N = 64
  return (2u << 4) | (1u << 7) | (1u << 10) | ((kStepKV >> 3) << 17) | ((kTileQ >> 4) << 24);
}

// Bounded wait for this warp's turn on the special-function unit; a finished peer never blocks us.
__device__ __forceinline__ bool wait_turn(uint32_t bar, uint32_t parity, volatile unsigned char* peer_done,
                                          volatile int* abort_flag, int code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 8; ++i)
      if (ptx::mbar_try_wait(bar, parity)) return true;
    if (*peer_done != 0) return true;
    if (*abort_flag != 0) return false;
    if (clock64() - t0 > kWaitCycles) {
      atomicCAS(const_cast<int*>(abort_flag), 0, code);
      return false;
    }
  }
}

// One softmax warpgroup: thread `row` (0..127) of tile `tile`; n_steps 64-key steps.
//
// The exponentials are the scarcest resource (16 per clock per SM, four per scheduler), and each
// scheduler hosts one warp of either tile.  The two warps take turns on it: a warp evaluates its 64
// exponentials while its peer stores P, fetches its next scores and finds their maximum, then hands
// over.  Without the hand-over both warps reach their exponentials together and the unit idles while
// both do the rest.
template <int D, int PV_MODE, int OUT_DTYPE>
__device__ __forceinline__ void softmax_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                             volatile int* abort_flag, volatile unsigned char* done_flags,
                                             int tile, int row, int n_steps, int q_row0, int b, int h, int h_kv) {
  const int wq = row >> 5;
  const uint32_t bar_my_turn = bars + 8 * (kBarTurn + tile * 4 + wq);
  const uint32_t bar_peer_turn = bars + 8 * (kBarTurn + (tile ^ 1) * 4 + wq);
  volatile unsigned char* peer_done = done_flags + (tile ^ 1) * 4 + wq;
  constexpr bool kF16Acc = (PV_MODE == SAGE_B200_PV_F16);
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  const uint32_t t_tile = tmem_base + lane_base + tile * 256;
  const uint32_t t_o = t_tile + 128;
  const uint32_t bar_pv_done = bars + 8 * (kBarPvDone + tile);

  const int q_row = q_row0 + row;
  float q_sc;
  {
    int g = (p.gran == SAGE_B200_GRAN_PER_THREAD) ? (q_row / p.warp_q) * 8 + (q_row & 7) : q_row / p.warp_q;
    if (g >= p.q_groups) g = p.q_groups - 1;
    q_sc = p.q_scale[(static_cast<int64_t>(b) * p.heads_q + h) * p.q_groups + g];
  }
  const float* ks_base = p.k_scale + (static_cast<int64_t>(b) * p.heads_kv + h_kv) * p.k_groups;
  const bool per_thread = (p.gran == SAGE_B200_GRAN_PER_THREAD);
  // k_scales of one step: four entries (per-thread grouping) or one (per-block); fetched one step ahead
  // (volatile, so that the load stays where it is written - a full step ahead of its use)
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
  float4 ks_next = load_scales(0);

#ifdef SAGE_TRACE
  long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long tprev = clock64();
#define SAGE_PH(k) do { const long long tn_ = clock64(); tacc[k] += tn_ - tprev; tprev = tn_; } while (0)
#else
#define SAGE_PH(k) do {} while (0)
#endif
  float m_run = -INFINITY;     // true running maximum (base 2, scaled)
  float m_used = -INFINITY;    // reference point P and O are expressed against
  float d_sum = 0.0f;
  bool ok = true;

#pragma unroll 1
  for (int i = 0; i < n_steps; ++i) {
    const int buf = i & 1;
    const int k0 = i * kStepKV;
    const uint32_t t_s = t_tile + buf * kStepKV;
    SAGE_PH(7);
    const float4 ks = ks_next;
    if (i + 1 < n_steps) ks_next = load_scales(i + 1);
    float a[4];
    a[0] = p.scale_log2 * (q_sc * ks.x);
    a[1] = p.scale_log2 * (q_sc * ks.y);
    a[2] = p.scale_log2 * (q_sc * ks.z);
    a[3] = p.scale_log2 * (q_sc * ks.w);
    SAGE_PH(0);
    ok = wait_bar_warp(bars + 8 * (kBarSFull + tile * 2 + buf), (i >> 1) & 1, abort_flag, 10 + tile);
    if (!ok) break;
    ptx::tc_fence_after();
    SAGE_PH(1);

    uint32_t s[64];
    ptx::tmem_ld32<0>(t_s + 0, s);
    ptx::tmem_ld32<32>(t_s + 32, s);
    ptx::tmem_wait_ld();
    SAGE_PH(2);

    const bool need_mask = (k0 + kStepKV > p.len_kv) || (p.causal && (k0 + kStepKV - 1 > q_row0));
    float m_blk = -INFINITY;
    if (!need_mask) {
      // X = float(S) + 1.5*2^23 without a conversion: |S| < 2^22, so adding S to the bit pattern of
      // 1.5*2^23 is exact.  X is monotonic in S: the maximum is taken on X per scale class
      // (three-input max) and mapped back through the class's constant.
#pragma unroll
      for (int c = 0; c < 64; ++c) s[c] += kMagicI;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float v[16];                                   // class t owns columns 2t + 8i, 2t + 8i + 1
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          v[2 * u] = __uint_as_float(s[2 * t + 8 * u]);
          v[2 * u + 1] = __uint_as_float(s[2 * t + 8 * u + 1]);
        }
        float mx = v[0];
#pragma unroll
        for (int u = 1; u < 15; u += 2) mx = ptx::max3(mx, v[u], v[u + 1]);
        mx = fmaxf(mx, v[15]);
        m_blk = fmaxf(m_blk, (mx - kMagicF) * a[t]);
      }
    } else {
      // diagonal or ragged step: scale first, mask to -inf, keep the scaled values in place
      const int lim_causal = p.causal ? (q_row - k0) : kStepKV;     // columns <= lim are visible
      const int lim = min(lim_causal, p.len_kv - k0 - 1);
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        float x = static_cast<float>(static_cast<int>(s[c])) * a[(c & 7) >> 1];
        x = (c <= lim) ? x : -INFINITY;
        m_blk = fmaxf(m_blk, x);
        s[c] = __float_as_uint(x);
      }
    }
    m_run = fmaxf(m_run, m_blk);

    // choose the reference point and the factor by which earlier work must shrink
    float alpha = 1.0f;
    bool rescale = false;
    if (i == 0) {
      m_used = m_run;
    } else {
      const float grow = m_run - m_used;
      if (kF16Acc ? (grow > 0.0f) : (grow > kLazyRescale)) {
        alpha = ptx::ex2(m_used - m_run);
        m_used = m_run;
        rescale = true;
      }
    }
    // a row that has seen nothing visible yet keeps a finite reference so that 2^(-inf - m) = 0
    const float m_ref = (m_used == -INFINITY) ? 0.0f : m_used;

    if (i > 0 && __any_sync(0xffffffffu, rescale)) {
      // O holds the sum through step i-1: its P.V must have retired before O is touched
      ok = wait_bar_warp(bar_pv_done, (i - 1) & 1, abort_flag, 20 + tile);
      if (!ok) break;
      ptx::tc_fence_after();
      if constexpr (kF16Acc) {
        // O is fp16 (one value per column); the factor is rounded to fp16 as the reference does
        // (update_mdo<..., true>, attn_utils.cuh:313-336)
        const __half a16 = __float2half_rn(alpha);
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t o[32];
          ptx::tmem_ld32<0>(t_o + c0, o);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int u = 0; u < 32; ++u)
            o[u] = __half_as_ushort(__hmul(__ushort_as_half(static_cast<unsigned short>(o[u] & 0xffffu)), a16));
          ptx::tmem_st32<0>(t_o + c0, o);
        }
      } else {
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t o[32];
          ptx::tmem_ld32<0>(t_o + c0, o);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int u = 0; u < 32; ++u) o[u] = __float_as_uint(__uint_as_float(o[u]) * alpha);
          ptx::tmem_st32<0>(t_o + c0, o);
        }
      }
      ptx::tmem_wait_st();
    }

    SAGE_PH(3);
#ifdef SAGE_TURNS
    // tile 0 goes first: its k-th turn follows the peer's (k-1)-th hand-over, tile 1's k-th follows
    // tile 0's k-th
    ok = __all_sync(0xffffffffu, wait_turn(bar_my_turn, tile == 0 ? ((i & 1) ^ 1) : (i & 1), peer_done, abort_flag, 70 + tile));
    if (!ok) break;
#endif
    SAGE_PH(4);

    // P = 2^(S*a - m), packed to fp16 pairs in place
    float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
    if (!need_mask) {
      // p = 2^(X*a + neg) with neg = -(1.5*2^23*a + m); two columns of one class per packed FMA
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
        float x0, x1, x2, x3;
        ptx::unpack2(e0, x0, x1);
        ptx::unpack2(e1, x2, x3);
        const float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1), p2 = ptx::ex2(x2), p3 = ptx::ex2(x3);
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
    SAGE_PH(5);
#ifdef SAGE_TURNS
    __syncwarp();
    if ((row & 31) == 0) ptx::mbar_arrive(bar_peer_turn);
#endif

    ptx::tmem_st32<0>(t_s, s);
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
    ptx::mbar_arrive(bars + 8 * (kBarPFull + tile * 2 + buf));
    SAGE_PH(6);
  }
#ifdef SAGE_TRACE
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (row & 31) == 0) {
    for (int k = 0; k < 8; ++k) p.trace[(tile * 4 + wq) * 8 + k] = tacc[k];
  }
#endif

  __syncwarp();
  if ((row & 31) == 0) done_flags[tile * 4 + wq] = 1;
  if (ok && n_steps > 0) {
    // A parity wait is only meaningful within one phase of the barrier's current phase; the per-step
    // barrier may be two phases behind here, so the end of the tile has a barrier of its own.
    ok = wait_bar_warp(bars + 8 * (kBarOFinal + tile), 0, abort_flag, 40 + tile);
    if (ok) ptx::tc_fence_after();
  }
  if (ok && n_steps > 0) {
    const float inv = ptx::rcp(d_sum);
    const bool store = q_row < p.len_q;
    unsigned short* orow = static_cast<unsigned short*>(p.out) + b * p.os_b + h * p.os_h + q_row * p.os_n;
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t o[32];
      ptx::tmem_ld32<0>(t_o + c0, o);
      ptx::tmem_wait_ld();
      uint32_t w[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        if constexpr (kF16Acc) {
          // normalise in fp32, round to fp16 (the accumulator type, normalize_d in attn_utils.cuh:565-567),
          // then to the output type
          const float lo = __half2float(__ushort_as_half(static_cast<unsigned short>(o[2 * u] & 0xffffu)));
          const float hi = __half2float(__ushort_as_half(static_cast<unsigned short>(o[2 * u + 1] & 0xffffu)));
          w[u] = pack_out<OUT_DTYPE>(__half2float(__float2half_rn(lo * inv)), __half2float(__float2half_rn(hi * inv)));
        } else {
          w[u] = pack_out<OUT_DTYPE>(__uint_as_float(o[2 * u]) * inv, __uint_as_float(o[2 * u + 1]) * inv);
        }
      }
      if (store) {
#pragma unroll
        for (int u = 0; u < 16; u += 4)
          *reinterpret_cast<uint4*>(orow + c0 + 2 * u) = make_uint4(w[u], w[u + 1], w[u + 2], w[u + 3]);
      }
    }
    if (p.lse != nullptr && store)
      p.lse[(static_cast<int64_t>(b) * p.heads_q + h) * p.len_q + q_row] = ptx::lg2(d_sum) + m_used;
  }
  ptx::tc_fence_before();
}

template <int D, int PV_MODE, int OUT_DTYPE>
__global__ void __launch_bounds__(kAttnThreads, 1)
sage_attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using Plan = SmemPlan<D>;
  constexpr bool kF16Acc = (PV_MODE == SAGE_B200_PV_F16);
  static_assert(PV_MODE != SAGE_B200_PV_F16_F32, "the two-level accumulate mode uses the coupled kernel");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bars = smem_base + Plan::kBarOff;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + Plan::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + Plan::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int h_kv = h / (p.heads_q / p.heads_kv);
  // causal: the heaviest tiles (largest query index) go first
  const int pair = p.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int q0 = pair * 2 * kTileQ;

  // another CTA of this launch already gave up: do not queue more bounded waits behind it
  if (launch_aborted(p)) return;

  int n_steps[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = q0 + t * kTileQ;
    const int kv_end = p.causal ? min(p.len_kv, r0 + kTileQ) : p.len_kv;
    n_steps[t] = (r0 < p.len_q) ? (kv_end + kStepKV - 1) / kStepKV : 0;
  }
  const int n_max = max(n_steps[0], n_steps[1]);
  const int n_stages = (n_max + 1) / 2;

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
    for (int t = 0; t < 4; ++t) {
      ptx::mbar_init(bars + 8 * (kBarSFull + t), 1);
      ptx::mbar_init(bars + 8 * (kBarPFull + t), kTileQ);
    }
    ptx::mbar_init(bars + 8 * (kBarPvDone + 0), 1);
    ptx::mbar_init(bars + 8 * (kBarPvDone + 1), 1);
    ptx::mbar_init(bars + 8 * (kBarOFinal + 0), 1);
    ptx::mbar_init(bars + 8 * (kBarOFinal + 1), 1);
    for (int t = 0; t < 8; ++t) ptx::mbar_init(bars + 8 * (kBarTurn + t), 1);
    ptx::mbar_init(bars + 8 * kBarDrain, 1);
    *abort_flag = 0;
    abort_flag[1] = 0;   // per-tile "finished" flags, one byte per (tile, warp)
    abort_flag[2] = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 8) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    ptx::reg_inc<224>();
    const int tile = warp >> 2;
    softmax_role<D, PV_MODE, OUT_DTYPE>(p, bars, tmem_base, abort_flag,
                                        reinterpret_cast<volatile unsigned char*>(smem_gen + Plan::kMiscOff + 8), tile,
                                        threadIdx.x & 127, n_steps[tile], q0 + tile * kTileQ, b, h, h_kv);
  } else {
    ptx::reg_dec<56>();
    if (warp == 8 && lane == 0) {
      // ---------------- TMA producer ----------------
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      const uint32_t q_smem = smem_base + Plan::kQOff;
      ptx::mbar_arrive_expect_tx(bars + 8 * kBarQFull, 2 * Plan::kQBytes);
      ptx::tma_load_4d(q_smem, &tm_q, bars + 8 * kBarQFull, 0, q0, h, b);
      ptx::tma_load_4d(q_smem + Plan::kQBytes, &tm_q, bars + 8 * kBarQFull, 0, q0 + kTileQ, h, b);
      bool ok = true;
#pragma unroll 1
      for (int j = 0; j < n_stages && ok; ++j) {
        const int ks = j % kKStages, vs = j % kVStages;
        ok = wait_bar(bars + 8 * (kBarKEmpty + ks), ((j / kKStages) & 1) ^ 1, abort_flag, 50);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bars + 8 * (kBarKFull + ks), Plan::kKBytes);
        ptx::tma_load_4d(smem_base + Plan::kKOff + ks * Plan::kKBytes, &tm_k, bars + 8 * (kBarKFull + ks), 0,
                         j * kStageKV, h_kv, b);
        ok = wait_bar(bars + 8 * (kBarVEmpty + vs), ((j / kVStages) & 1) ^ 1, abort_flag, 51);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bars + 8 * (kBarVFull + vs), Plan::kVBytes);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn)
          ptx::tma_load_4d(smem_base + Plan::kVOff + vs * Plan::kVBytes + pn * (kStageKV * 128), &tm_v,
                           bars + 8 * (kBarVFull + vs), pn * 64, j * kStageKV, h_kv, b);
      }
      if (!ok) {
        // leave no copy in flight behind us: wait (bounded) for what was issued
        for (int s = 0; s < kKStages; ++s)
          for (int i = 0; i < 4096 && !ptx::mbar_try_wait(bars + 8 * (kBarKFull + s), 0) &&
                          !ptx::mbar_try_wait(bars + 8 * (kBarKFull + s), 1); ++i) {}
      }
    } else if (warp == 9) {
      // ---------------- MMA issuer ----------------
      // The whole warp runs this loop and one elected lane issues: operands that are computed in
      // converged code stay in uniform registers, which tcgen05.mma and tcgen05.commit read directly.
      constexpr int kRowBytesQK = (D == 64) ? 64 : 128;
      constexpr int kStepsQK = kRowBytesQK / 32;              // int8: 32 bytes of K per instruction
      const uint32_t idq = idesc_qk64();
      const uint32_t idp = idesc_pv<D, kF16Acc>();
      // Descriptors differ only in their 14-bit start-address field (units of 16 bytes), which never
      // carries out of the field for shared-memory addresses: build them once, then add offsets.
      const uint64_t q_desc0 = desc_kmajor<kRowBytesQK>(smem_base + Plan::kQOff);
      const uint64_t k_desc0 = desc_kmajor<kRowBytesQK>(smem_base + Plan::kKOff);
      const uint64_t v_desc0 = desc_mnmajor(smem_base + Plan::kVOff, kStageKV * 128);

      // S[t][step & 1] = Q_t . K(step)^T, 64 keys
      auto issue_qk = [&](int t, int step, uint32_t commit_bar) {
        const int stage = (step >> 1) % kKStages;
        const uint32_t d_t = tmem_base + t * 256 + (step & 1) * kStepKV;
        const uint64_t da0 = q_desc0 + static_cast<uint64_t>((t * Plan::kQBytes) >> 4);
        const uint64_t db0 = k_desc0 + static_cast<uint64_t>((stage * Plan::kKBytes + (step & 1) * kStepKV * kRowBytesQK) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kStepsQK; ++s)
            ptx::mma_i8_ss(d_t, da0 + static_cast<uint64_t>(s * 2), db0 + static_cast<uint64_t>(s * 2), idq, s != 0);
          ptx::tc_commit(commit_bar);
        }
        __syncwarp();
      };
      // O_t (+)= P(step) . V(step): 16 keys per instruction = 8 packed columns of P, 2 KB of every V panel
      auto issue_pv = [&](int t, int step, uint32_t commit_bar, bool last) {
        const int stage = (step >> 1) % kVStages;
        const uint32_t d_t = tmem_base + t * 256 + 128;
        const uint32_t a_t = tmem_base + t * 256 + (step & 1) * kStepKV;
        const uint64_t db0 = v_desc0 + static_cast<uint64_t>((stage * Plan::kVBytes + (step & 1) * kStepKV * 128) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kStepKV / 16; ++s)
            ptx::mma_f16_ts(d_t, a_t + s * 8, db0 + static_cast<uint64_t>(s * 128), idp, (step > 0 || s != 0) ? 1u : 0u);
          ptx::tc_commit(commit_bar);
          if (last) ptx::tc_commit(bars + 8 * (kBarOFinal + t));
        }
        __syncwarp();
      };
      auto commit_only = [&](uint32_t bar) {
        if (ptx::elect_one()) ptx::tc_commit(bar);
        __syncwarp();
      };

      bool ok = wait_bar_warp(bars + 8 * kBarQFull, 0, abort_flag, 60);
      if (ok && n_max > 0) ok = wait_bar_warp(bars + 8 * (kBarKFull + 0), 0, abort_flag, 61);
      if (ok && n_max > 0) {
        ptx::tc_fence_after();
        for (int st = 0; st < 2; ++st) {
          for (int t = 0; t < 2; ++t) {
            if (st < n_steps[t]) {
              issue_qk(t, st, bars + 8 * (kBarSFull + t * 2 + st));
            }
          }
        }
        commit_only(bars + 8 * (kBarKEmpty + 0));
      }
#ifdef SAGE_TRACE
      long long macc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      long long mprev = clock64();
#define MMA_PH(k) do { const long long tn_ = clock64(); macc[k] += tn_ - mprev; mprev = tn_; } while (0)
#else
#define MMA_PH(k) do {} while (0)
#endif
#pragma unroll 1
      for (int i = 0; i < n_max && ok; ++i) {
        const int blk = i >> 1;
        const int vs = blk % kVStages;
        const int nxt = i + 2;                       // the step whose Q.K^T reuses this S buffer
        const int ks = (nxt >> 1) % kKStages;
        if ((i & 1) == 0) {
          ok = wait_bar_warp(bars + 8 * (kBarVFull + vs), (blk / kVStages) & 1, abort_flag, 62);
          if (!ok) break;
          if (nxt < n_max) {
            ok = wait_bar_warp(bars + 8 * (kBarKFull + ks), ((nxt >> 1) / kKStages) & 1, abort_flag, 63);
            if (!ok) break;
          }
        }
        for (int t = 0; t < 2 && ok; ++t) {
          if (i < n_steps[t]) {
            MMA_PH(0);
            ok = wait_bar_warp(bars + 8 * (kBarPFull + t * 2 + (i & 1)), (i >> 1) & 1, abort_flag, 64 + t);
            if (!ok) break;
            ptx::tc_fence_after();
            MMA_PH(1 + 3 * t);
            issue_pv(t, i, bars + 8 * (kBarPvDone + t), i == n_steps[t] - 1);
            MMA_PH(2 + 3 * t);
            if (nxt < n_steps[t]) {
              issue_qk(t, nxt, bars + 8 * (kBarSFull + t * 2 + (i & 1)));
            }
            MMA_PH(3 + 3 * t);
          }
        }
        if (!ok) break;
        MMA_PH(0);
        if ((i & 1) == 1 || i == n_max - 1) commit_only(bars + 8 * (kBarVEmpty + vs));
        if ((i & 1) == 1 && nxt < n_max) commit_only(bars + 8 * (kBarKEmpty + ks));
        MMA_PH(7);
      }
#ifdef SAGE_TRACE
      if (p.trace != nullptr && lane == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
        for (int k = 0; k < 8; ++k) p.trace[64 + k] = macc[k];
#endif
      // everything this thread issued must have retired before tensor memory is released
      commit_only(bars + 8 * kBarDrain);
      for (int i = 0; i < (1 << 20) && !ptx::mbar_try_wait(bars + 8 * kBarDrain, 0); ++i) {}
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (warp == 8) ptx::tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && *abort_flag != 0) publish_abort(p, *abort_flag);
}

}  // namespace v2
}  // namespace sage
