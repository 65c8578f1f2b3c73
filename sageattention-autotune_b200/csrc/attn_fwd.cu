// SageAttention core for B200 (sm_100a): int8 Q.K^T and fp16 P.V on tcgen05 tensor cores with
// accumulators in tensor memory, TMA-staged operands, online softmax in two softmax warpgroups.
//
// It replaces the reference's qk_int8_sv_f16_attn_kernel
// (csrc/qattn/qk_int8_sv_f16_kernel_sm80.cuh:61-657) and its launcher
// (csrc/qattn/qk_int8_sv_f16_launch_sm80.cuh:177-308); the arithmetic follows the same order:
// S = int32(Q.K^T) -> scale by q_scale*k_scale*sm_scale*log2(e) -> running max in base 2 ->
// P = 2^(S*a - m) rounded to fp16 -> O += P.V -> O / sum(P).
//
// One CTA = one (batch, q-head) and 256 consecutive query rows = two 128-row tiles.
//   warps 0-3   softmax warpgroup of tile 0 (thread t owns query row t: TMEM lane t)
//   warps 4-7   softmax warpgroup of tile 1
//   warp  8     TMA producer (one elected lane) and owner of the TMEM allocation
//   warp  9     MMA issuer (one elected lane)
//   warps 10-11 idle (they complete the third warpgroup so that setmaxnreg can be used)
// Tensor memory (512 columns): per tile 128 columns for S (int32); P (fp16, two keys per
// column) overwrites columns 0-63 of S; 128 more columns hold O.  An fp16 accumulator occupies
// one column per element (value in the low half), so the "fp16" mode keeps O as D such columns,
// and the "fp16+fp32" mode computes each block's partial product 64 channels at a time into
// columns 64-127 of S and folds it into the fp32 O before the next 64 channels are issued.
// K/V blocks of 128 keys are shared by both tiles, so each byte of K and V is fetched once per
// 256 query rows.
//
// Scales: thread t reads its own q_scale and, per 64 keys, the four k_scales of the reference's
// per-thread grouping (key c uses entry (c%8)/2), qk_int8_sv_f16_kernel_sm80.cuh:116-126.  Which
// entry applies to a column is a compile-time function of the unrolled column index, so the
// dequantisation costs nothing beyond the FMA that feeds ex2.
//
// Every wait on an mbarrier is bounded: when it runs out the CTA raises an abort flag, all
// roles leave their loops, tensor memory is released and a code is written to the caller's status
// word.  Nothing traps.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace sage {

constexpr int kTileQ = 128;
constexpr int kBlockKV = 128;
constexpr int kAttnThreads = 384;
constexpr int kKStages = 3;
constexpr int kVStages = 3;
constexpr long long kWaitCycles = 4000000000LL;   // about two seconds of SM clock
constexpr float kLog2e = 1.44269504088896340736f;
constexpr float kMagicF = 12582912.0f;            // 1.5 * 2^23
constexpr uint32_t kMagicI = 0x4B400000u;
constexpr float kLazyRescale = 8.0f;              // fp32 accumulators: rescale O only if max grew by 2^8

struct AttnParams {
  const float* q_scale;
  const float* k_scale;
  void* out;
  float* lse;
  int32_t* status;
  int len_q, len_kv, heads_q, heads_kv;
  int q_groups, k_groups;       // scale entries per head
  int warp_q;                    // WARPQ (per-thread) or BLKQ (per-block)
  int gran;
  int causal;
  float scale_log2;              // sm_scale * log2(e)
  int64_t os_b, os_h, os_n;
};

enum BarIdx {
  kBarQFull = 0,
  kBarKFull = 1,                          // kKStages
  kBarKEmpty = kBarKFull + kKStages,
  kBarVFull = kBarKEmpty + kKStages,      // kVStages
  kBarVEmpty = kBarVFull + kVStages,
  kBarSFull = kBarVEmpty + kVStages,      // 2
  kBarPFull = kBarSFull + 2,              // 2
  kBarPvDone = kBarPFull + 2,             // 2
  kBarSFree = kBarPvDone + 2,             // 2
  kBarDrain = kBarSFree + 2,
  kNumBars = kBarDrain + 1
};

template <int D>
struct SmemPlan {
  static constexpr int kQBytes = kTileQ * D;                 // int8
  static constexpr int kKBytes = kBlockKV * D;               // int8
  static constexpr int kVBytes = kBlockKV * D * 2;           // fp16
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + 2 * kQBytes;
  static constexpr int kVOff = kKOff + kKStages * kKBytes;
  static constexpr int kBarOff = kVOff + kVStages * kVBytes;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;             // slack for manual 1024-byte alignment
};

// Bounded mbarrier wait.  Returns false if the CTA is aborting.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (ptx::mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (clock64() - t0 > kWaitCycles) {
      atomicCAS(const_cast<int*>(abort_flag), 0, code);
      return false;
    }
  }
}

// Same, for code that goes on to warp-collective tcgen05.ld/st: the verdict is made warp-uniform.
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  return __all_sync(0xffffffffu, wait_bar(bar, parity, abort_flag, code));
}

// K-major operand tile whose rows are ROW_BYTES wide (64 -> 64-byte swizzle, 128 -> 128-byte swizzle)
template <int ROW_BYTES>
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t smem_addr) {
  constexpr uint64_t layout = (ROW_BYTES == 128) ? 2 : 4;
  constexpr uint64_t sbo = (8 * ROW_BYTES) >> 4;            // 8 rows
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (sbo << 32) |
         (uint64_t(1) << 46) | (layout << 61);
}
// MN-major operand (V as [keys][64 channels] panels, 128-byte swizzle): 8 keys = 1024 bytes apart,
// next 64-channel panel `panel_bytes` apart
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t smem_addr, uint32_t panel_bytes) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(panel_bytes >> 4) << 16) |
         (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}

__host__ __device__ constexpr uint32_t idesc_qk() {
  // int8 x int8 -> int32, both K-major, M = 128, N = 128
  return (2u << 4) | (1u << 7) | (1u << 10) | ((kBlockKV >> 3) << 17) | ((kTileQ >> 4) << 24);
}
template <int D, bool F16_ACC>
__host__ __device__ constexpr uint32_t idesc_pv() {
  // fp16 x fp16 -> fp32 (or fp16), A from tensor memory, B MN-major, M = 128, N = D
  return ((F16_ACC ? 0u : 1u) << 4) | (0u << 7) | (0u << 10) | (1u << 16) | ((uint32_t(D) >> 3) << 17) |
         ((kTileQ >> 4) << 24);
}

template <int OUT_DTYPE>
__device__ __forceinline__ uint32_t pack_out(float lo, float hi) {
  if constexpr (OUT_DTYPE == SAGE_B200_BF16) return ptx::pack_bf16x2(lo, hi);
  else return ptx::pack_f16x2(lo, hi);
}

__device__ __forceinline__ int k_class(int c) { return ((c >> 6) << 2) | ((c & 7) >> 1); }

// One softmax warpgroup: thread `row` (0..127) of tile `tile`.
template <int D, int PV_MODE, int OUT_DTYPE>
__device__ __forceinline__ void softmax_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                             volatile int* abort_flag, int tile, int row, int n_blocks,
                                             int q_row0, int b, int h, int h_kv) {
  constexpr bool kF16Acc = (PV_MODE == SAGE_B200_PV_F16);
  constexpr bool kInstBuf = (PV_MODE == SAGE_B200_PV_F16_F32);
  const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
  const uint32_t t_s = tmem_base + lane_base + tile * 256;
  const uint32_t t_p = t_s;
  const uint32_t t_t = t_s + 64;
  const uint32_t t_o = t_s + 128;
  const uint32_t bar_s_full = bars + 8 * (kBarSFull + tile);
  const uint32_t bar_p_full = bars + 8 * (kBarPFull + tile);
  const uint32_t bar_pv_done = bars + 8 * (kBarPvDone + tile);
  const uint32_t bar_s_free = bars + 8 * (kBarSFree + tile);

  const int q_row = q_row0 + row;
  float q_sc;
  {
    int g = (p.gran == SAGE_B200_GRAN_PER_THREAD) ? (q_row / p.warp_q) * 8 + (q_row & 7) : q_row / p.warp_q;
    if (g >= p.q_groups) g = p.q_groups - 1;
    q_sc = p.q_scale[(static_cast<int64_t>(b) * p.heads_q + h) * p.q_groups + g];
  }
  const float* ks_base = p.k_scale + (static_cast<int64_t>(b) * p.heads_kv + h_kv) * p.k_groups;

  float m_run = -INFINITY;     // true running maximum (base 2, scaled)
  float m_used = -INFINITY;    // reference point P and O are expressed against
  float d_sum = 0.0f;
  bool ok = true;

#pragma unroll 1
  for (int j = 0; j < n_blocks; ++j) {
    const int k0 = j * kBlockKV;
    // the eight dequantisation constants of this block
    float a[8];
    if (p.gran == SAGE_B200_GRAN_PER_THREAD) {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int g = j * 8 + t;
        a[t] = (g < p.k_groups) ? __ldg(ks_base + g) : 0.0f;
      }
    } else {
      const float s0 = (2 * j < p.k_groups) ? __ldg(ks_base + 2 * j) : 0.0f;
      const float s1 = (2 * j + 1 < p.k_groups) ? __ldg(ks_base + 2 * j + 1) : 0.0f;
#pragma unroll
      for (int t = 0; t < 4; ++t) { a[t] = s0; a[4 + t] = s1; }
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) a[t] = p.scale_log2 * (q_sc * a[t]);

    ok = wait_bar_warp(bar_s_full, j & 1, abort_flag, 10 + tile);
    if (!ok) break;
    ptx::tc_fence_after();

    uint32_t s[128];
    ptx::tmem_ld32<0>(t_s + 0, s);
    ptx::tmem_ld32<32>(t_s + 32, s);
    ptx::tmem_ld32<64>(t_s + 64, s);
    ptx::tmem_ld32<96>(t_s + 96, s);
    ptx::tmem_wait_ld();

    const bool need_mask = (k0 + kBlockKV > p.len_kv) || (p.causal && (k0 + kBlockKV - 1 > q_row0));
    float m_blk = -INFINITY;
    if (!need_mask) {
      int mx[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) mx[t] = INT_MIN;
#pragma unroll
      for (int c = 0; c < 128; ++c) mx[k_class(c)] = max(mx[k_class(c)], static_cast<int>(s[c]));
#pragma unroll
      for (int t = 0; t < 8; ++t) m_blk = fmaxf(m_blk, static_cast<float>(mx[t]) * a[t]);
    } else {
      // diagonal or ragged block: scale first, mask to -inf, keep the scaled values in place
      const int lim_causal = p.causal ? (q_row - k0) : kBlockKV;     // columns <= lim are visible
      const int lim_len = p.len_kv - k0 - 1;
      const int lim = min(lim_causal, lim_len);
#pragma unroll
      for (int c = 0; c < 128; ++c) {
        float x = static_cast<float>(static_cast<int>(s[c])) * a[k_class(c)];
        x = (c <= lim) ? x : -INFINITY;
        m_blk = fmaxf(m_blk, x);
        s[c] = __float_as_uint(x);
      }
    }
    m_run = fmaxf(m_run, m_blk);

    // choose the reference point and the factor by which earlier work must shrink
    float alpha = 1.0f;
    bool rescale = false;
    if (j == 0) {
      m_used = m_run;
    } else {
      const float grow = m_run - m_used;
      if ((kF16Acc || kInstBuf) ? (grow > 0.0f) : (grow > kLazyRescale)) {
        alpha = ptx::ex2(m_used - m_run);
        m_used = m_run;
        rescale = true;
      }
    }
    // a row that has seen nothing visible yet keeps a finite reference so that 2^(-inf - m) = 0
    const float m_ref = (m_used == -INFINITY) ? 0.0f : m_used;

    if constexpr (!kInstBuf) {
      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
        ok = wait_bar_warp(bar_pv_done, (j - 1) & 1, abort_flag, 20 + tile);
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
            for (int i = 0; i < 32; ++i) {
              const __half v = __hmul(__ushort_as_half(static_cast<unsigned short>(o[i] & 0xffffu)), a16);
              o[i] = __half_as_ushort(v);
            }
            ptx::tmem_st32<0>(t_o + c0, o);
          }
        } else {
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            ptx::tmem_ld32<0>(t_o + c0, o);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            ptx::tmem_st32<0>(t_o + c0, o);
          }
        }
        ptx::tmem_wait_st();
      }
    }

    // P = 2^(S*a - m), packed to fp16 pairs in place
    float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
    if (!need_mask) {
      float neg[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) neg[t] = fmaf(-kMagicF, a[t], -m_ref);
#pragma unroll
      for (int c = 0; c < 128; c += 4) {
        const float x0 = __uint_as_float(s[c + 0] + kMagicI), x1 = __uint_as_float(s[c + 1] + kMagicI);
        const float x2 = __uint_as_float(s[c + 2] + kMagicI), x3 = __uint_as_float(s[c + 3] + kMagicI);
        const float p0 = ptx::ex2(fmaf(x0, a[k_class(c + 0)], neg[k_class(c + 0)]));
        const float p1 = ptx::ex2(fmaf(x1, a[k_class(c + 1)], neg[k_class(c + 1)]));
        const float p2 = ptx::ex2(fmaf(x2, a[k_class(c + 2)], neg[k_class(c + 2)]));
        const float p3 = ptx::ex2(fmaf(x3, a[k_class(c + 3)], neg[k_class(c + 3)]));
        sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
        s[c / 2 + 0] = ptx::pack_f16x2(p0, p1);
        s[c / 2 + 1] = ptx::pack_f16x2(p2, p3);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 128; c += 2) {
        const float p0 = ptx::ex2(__uint_as_float(s[c + 0]) - m_ref);
        const float p1 = ptx::ex2(__uint_as_float(s[c + 1]) - m_ref);
        sum0 += p0; sum1 += p1;
        s[c / 2] = ptx::pack_f16x2(p0, p1);
      }
    }
    d_sum = d_sum * alpha + ((sum0 + sum1) + (sum2 + sum3));

    ptx::tmem_st32<0>(t_p + 0, s);
    ptx::tmem_st32<32>(t_p + 32, s);
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
    ptx::mbar_arrive(bar_p_full);

    if constexpr (kInstBuf) {
      // "fp16+fp32": this block's P.V is accumulated in fp16 from zero, 64 channels at a time, and
      // folded into the fp32 O (compute_fp16_sv_permuted_inst_buf, attn_utils.cuh:447-518)
      const bool any_rescale = __any_sync(0xffffffffu, rescale);
#pragma unroll 1
      for (int ch = 0; ch < D / 64 && ok; ++ch) {
        ok = wait_bar_warp(bar_pv_done, (j * (D / 64) + ch) & 1, abort_flag, 30 + tile);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t t16[32];
          uint32_t o[32];
          ptx::tmem_ld32<0>(t_t + c0, t16);
          if (j > 0) ptx::tmem_ld32<0>(t_o + ch * 64 + c0, o);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float acc = (j > 0) ? __uint_as_float(o[i]) : 0.0f;
            if (any_rescale) acc *= alpha;
            o[i] = __float_as_uint(ptx::add_f32_f16(acc, static_cast<unsigned short>(t16[i] & 0xffffu)));
          }
          ptx::tmem_st32<0>(t_o + ch * 64 + c0, o);
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_s_free);
      }
      if (!ok) break;
    }
  }

  if (ok && n_blocks > 0) {
    if constexpr (!kInstBuf) {
      ok = wait_bar_warp(bar_pv_done, (n_blocks - 1) & 1, abort_flag, 40 + tile);
      if (ok) ptx::tc_fence_after();
    }
  }
  if (ok && n_blocks > 0) {
    const float inv = ptx::rcp(d_sum);
    const bool store = q_row < p.len_q;
    unsigned short* orow = static_cast<unsigned short*>(p.out) + b * p.os_b + h * p.os_h + q_row * p.os_n;
    if constexpr (kF16Acc) {
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t o[32];
        ptx::tmem_ld32<0>(t_o + c0, o);
        ptx::tmem_wait_ld();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          // normalise in fp32, round to fp16 (the accumulator type, normalize_d in attn_utils.cuh:565-567),
          // then to the output type
          const float lo = __half2float(__ushort_as_half(static_cast<unsigned short>(o[2 * i] & 0xffffu)));
          const float hi = __half2float(__ushort_as_half(static_cast<unsigned short>(o[2 * i + 1] & 0xffffu)));
          w[i] = pack_out<OUT_DTYPE>(__half2float(__float2half_rn(lo * inv)), __half2float(__float2half_rn(hi * inv)));
        }
        if (store) {
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<uint4*>(orow + c0 + 2 * i) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
        }
      }
    } else {
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
  constexpr bool kInstBuf = (PV_MODE == SAGE_B200_PV_F16_F32);
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
  if (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) return;

  int n_blk[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = q0 + t * kTileQ;
    int kv_end = p.causal ? min(p.len_kv, r0 + kTileQ) : p.len_kv;
    n_blk[t] = (r0 < p.len_q) ? (kv_end + kBlockKV - 1) / kBlockKV : 0;
  }
  const int n_max = max(n_blk[0], n_blk[1]);

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
      ptx::mbar_init(bars + 8 * (kBarPvDone + t), 1);
      ptx::mbar_init(bars + 8 * (kBarSFree + t), kTileQ);
    }
    ptx::mbar_init(bars + 8 * kBarDrain, 1);
    *abort_flag = 0;
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
    ptx::reg_inc<232>();
    const int tile = warp >> 2;
    softmax_role<D, PV_MODE, OUT_DTYPE>(p, bars, tmem_base, abort_flag, tile, threadIdx.x & 127, n_blk[tile],
                                        q0 + tile * kTileQ, b, h, h_kv);
  } else {
    ptx::reg_dec<40>();
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
      for (int j = 0; j < n_max && ok; ++j) {
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
        // leave no copy in flight behind us: wait (bounded by the hardware try_wait) for what was issued
        for (int s = 0; s < kKStages; ++s)
          for (int i = 0; i < 4096 && !ptx::mbar_try_wait(bars + 8 * (kBarKFull + s), 0) &&
                          !ptx::mbar_try_wait(bars + 8 * (kBarKFull + s), 1); ++i) {}
      }
    } else if (warp == 9 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr int kRowBytesQK = (D == 64) ? 64 : 128;
      constexpr int kPanelsQK = D / kRowBytesQK;              // 1 (2 for D = 256)
      constexpr int kStepsPerPanel = kRowBytesQK / 32;        // int8: 32 bytes of K per instruction
      const uint32_t q_smem = smem_base + Plan::kQOff;
      const uint32_t k_smem = smem_base + Plan::kKOff;
      const uint32_t v_smem = smem_base + Plan::kVOff;
      const uint32_t idq = idesc_qk();
      const uint32_t idp = idesc_pv<D, kF16Acc>();
      const uint32_t idp_chunk = idesc_pv<64, true>();

      auto issue_qk = [&](int t, int stage) {
        const uint32_t d_t = tmem_base + t * 256;
#pragma unroll
        for (int pn = 0; pn < kPanelsQK; ++pn) {
#pragma unroll
          for (int s = 0; s < kStepsPerPanel; ++s) {
            const uint32_t off = pn * (kTileQ * kRowBytesQK) + s * 32;
            const uint64_t da = desc_kmajor<kRowBytesQK>(q_smem + t * Plan::kQBytes + off);
            const uint64_t db = desc_kmajor<kRowBytesQK>(k_smem + stage * Plan::kKBytes + off);
            ptx::mma_i8_ss(d_t, da, db, idq, (pn | s) != 0);
          }
        }
      };
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t d_t = tmem_base + t * 256 + 128;
        const uint32_t a_t = tmem_base + t * 256;
#pragma unroll
        for (int s = 0; s < kBlockKV / 16; ++s) {
          // 16 keys per instruction: 8 packed columns of P, 16 rows (2 KB) of every V panel
          const uint64_t db = desc_mnmajor(v_smem + stage * Plan::kVBytes + s * 2048, kBlockKV * 128);
          ptx::mma_f16_ts(d_t, a_t + s * 8, db, idp, (accumulate || s != 0) ? 1u : 0u);
        }
      };
      // "fp16+fp32": one 64-channel panel of V at a time into the fp16 scratch columns
      auto issue_pv_chunk = [&](int t, int stage, int ch) {
        const uint32_t d_t = tmem_base + t * 256 + 64;
        const uint32_t a_t = tmem_base + t * 256;
#pragma unroll
        for (int s = 0; s < kBlockKV / 16; ++s) {
          const uint64_t db = desc_mnmajor(v_smem + stage * Plan::kVBytes + ch * (kBlockKV * 128) + s * 2048,
                                           kBlockKV * 128);
          ptx::mma_f16_ts(d_t, a_t + s * 8, db, idp_chunk, s != 0 ? 1u : 0u);
        }
      };

      bool ok = wait_bar(bars + 8 * kBarQFull, 0, abort_flag, 60);
      if (ok && n_max > 0) ok = wait_bar(bars + 8 * (kBarKFull + 0), 0, abort_flag, 61);
      if (ok && n_max > 0) {
        ptx::tc_fence_after();
        for (int t = 0; t < 2; ++t) {
          if (n_blk[t] > 0) {
            issue_qk(t, 0);
            ptx::tc_commit(bars + 8 * (kBarSFull + t));
          }
        }
        ptx::tc_commit(bars + 8 * (kBarKEmpty + 0));
      }
#pragma unroll 1
      for (int j = 0; j < n_max && ok; ++j) {
        const int vs = j % kVStages;
        const int nxt = j + 1;
        const int ks = nxt % kKStages;
        ok = wait_bar(bars + 8 * (kBarVFull + vs), (j / kVStages) & 1, abort_flag, 62);
        if (!ok) break;
        if (nxt < n_max) {
          ok = wait_bar(bars + 8 * (kBarKFull + ks), (nxt / kKStages) & 1, abort_flag, 63);
          if (!ok) break;
        }
        if constexpr (!kInstBuf) {
          for (int t = 0; t < 2 && ok; ++t) {
            if (j < n_blk[t]) {
              ok = wait_bar(bars + 8 * (kBarPFull + t), j & 1, abort_flag, 64 + t);
              if (!ok) break;
              ptx::tc_fence_after();
              issue_pv(t, vs, j > 0);
              ptx::tc_commit(bars + 8 * (kBarPvDone + t));
              if (nxt < n_blk[t]) {
                issue_qk(t, ks);
                ptx::tc_commit(bars + 8 * (kBarSFull + t));
              }
            }
          }
        } else {
          constexpr int kChunks = D / 64;
          for (int ch = 0; ch < kChunks && ok; ++ch) {
            for (int t = 0; t < 2 && ok; ++t) {
              if (j < n_blk[t]) {
                if (ch == 0) ok = wait_bar(bars + 8 * (kBarPFull + t), j & 1, abort_flag, 64 + t);
                else ok = wait_bar(bars + 8 * (kBarSFree + t), (j * kChunks + ch - 1) & 1, abort_flag, 66 + t);
                if (!ok) break;
                ptx::tc_fence_after();
                issue_pv_chunk(t, vs, ch);
                ptx::tc_commit(bars + 8 * (kBarPvDone + t));
              }
            }
          }
          for (int t = 0; t < 2 && ok; ++t) {
            if (nxt < n_blk[t]) {
              ok = wait_bar(bars + 8 * (kBarSFree + t), (j * kChunks + kChunks - 1) & 1, abort_flag, 68 + t);
              if (!ok) break;
              ptx::tc_fence_after();
              issue_qk(t, ks);
              ptx::tc_commit(bars + 8 * (kBarSFull + t));
            }
          }
        }
        if (!ok) break;
        ptx::tc_commit(bars + 8 * (kBarVEmpty + vs));
        if (nxt < n_max) ptx::tc_commit(bars + 8 * (kBarKEmpty + ks));
      }
      // everything this thread issued must have retired before tensor memory is released
      ptx::tc_commit(bars + 8 * kBarDrain);
      for (int i = 0; i < (1 << 20) && !ptx::mbar_try_wait(bars + 8 * kBarDrain, 0); ++i) {}
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (warp == 8) ptx::tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, *abort_flag) == 0) {
      p.status[1] = blockIdx.x;
      p.status[2] = blockIdx.y;
      p.status[3] = blockIdx.z;
    }
  }
}

// ------------------------------------------------------------------------------------------- host
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// (batch, heads, len, head_dim) tensor with element strides -> 4-D tensor map (d, n, h, b)
static int make_map(CUtensorMap* map, const void* base, int elem_bytes, int batch, int heads, int len,
                    int head_dim, const int64_t st[3], int box_d, int box_n, CUtensorMapSwizzle swz,
                    const char* what) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(SAGE_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  SAGE_REQUIRE(aligned16(base), "attn_fwd: %s must be 16-byte aligned", what);
  for (int i = 0; i < 3; ++i)
    SAGE_REQUIRE((st[i] * elem_bytes) % 16 == 0, "attn_fwd: %s strides must be multiples of 16 bytes", what);
  const cuuint64_t dims[4] = {cuuint64_t(head_dim), cuuint64_t(len), cuuint64_t(heads), cuuint64_t(batch)};
  // a dimension of extent 1 may carry any stride; give it a legal one
  const cuuint64_t strides[3] = {cuuint64_t(st[2]) * elem_bytes,
                                 cuuint64_t(heads > 1 ? st[1] : int64_t(head_dim)) * elem_bytes,
                                 cuuint64_t(batch > 1 ? st[0] : int64_t(head_dim)) * elem_bytes};
  const cuuint32_t box[4] = {cuuint32_t(box_d), cuuint32_t(box_n), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = (elem_bytes == 1) ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SAGE_B200_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with code %d", what, int(r));
  return SAGE_B200_OK;
}

template <int D, int PV_MODE, int OUT_DTYPE>
static int launch_attn(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p,
                       dim3 grid, cudaStream_t stream) {
  auto kern = sage_attn_fwd_kernel<D, PV_MODE, OUT_DTYPE>;
  cudaError_t attr_err = cudaSuccess;
  constexpr int smem = SmemPlan<D>::kDynamic;
  // the attribute is per device: set it for every device that launches
  static bool done[64] = {};
  static std::mutex mu;
  int dev = 0;
  SAGE_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (attr_err != cudaSuccess)
        return fail(SAGE_B200_ERR_CUDA, "cudaFuncSetAttribute(%d bytes) failed: %s", smem, cudaGetErrorString(attr_err));
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  kern<<<grid, kAttnThreads, smem, stream>>>(mq, mk, mv, p);
  SAGE_CUDA_TRY(cudaGetLastError());
  return SAGE_B200_OK;
}

template <int D, int PV_MODE>
static int launch_attn_out(int out_dtype, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                           const AttnParams& p, dim3 grid, cudaStream_t stream) {
  if (out_dtype == SAGE_B200_BF16) return launch_attn<D, PV_MODE, SAGE_B200_BF16>(mq, mk, mv, p, grid, stream);
  return launch_attn<D, PV_MODE, SAGE_B200_F16>(mq, mk, mv, p, grid, stream);
}

template <int D>
static int launch_attn_mode(int pv_accum, int out_dtype, const CUtensorMap& mq, const CUtensorMap& mk,
                            const CUtensorMap& mv, const AttnParams& p, dim3 grid, cudaStream_t stream) {
  switch (pv_accum) {
    case SAGE_B200_PV_F32: return launch_attn_out<D, SAGE_B200_PV_F32>(out_dtype, mq, mk, mv, p, grid, stream);
    case SAGE_B200_PV_F16: return launch_attn_out<D, SAGE_B200_PV_F16>(out_dtype, mq, mk, mv, p, grid, stream);
    default: return launch_attn_out<D, SAGE_B200_PV_F16_F32>(out_dtype, mq, mk, mv, p, grid, stream);
  }
}

}  // namespace sage

using namespace sage;

extern "C" int sage_b200_attn_fwd(const int8_t* q, const int8_t* k, const void* v, void* out,
                                  const float* q_scale, const float* k_scale, float* lse, int32_t* status,
                                  int out_dtype, int batch, int heads_q, int heads_kv, int len_q, int len_kv,
                                  int head_dim, const int64_t q_strides[3], const int64_t k_strides[3],
                                  const int64_t v_strides[3], const int64_t o_strides[3], int is_causal,
                                  float sm_scale, int blk_q, int blk_k, int warp_q, int warp_k,
                                  int granularity, int pv_accum, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  SAGE_REQUIRE(q && k && v && out && q_scale && k_scale, "attn_fwd: null pointer");
  SAGE_REQUIRE(q_strides && k_strides && v_strides && o_strides, "attn_fwd: null stride array");
  SAGE_REQUIRE(out_dtype == SAGE_B200_F16 || out_dtype == SAGE_B200_BF16, "attn_fwd: out_dtype must be fp16 or bf16");
  SAGE_REQUIRE(batch > 0 && heads_q > 0 && heads_kv > 0 && len_q > 0 && len_kv > 0, "attn_fwd: empty tensor");
  SAGE_REQUIRE(batch <= 65535 && heads_q <= 65535, "attn_fwd: batch/heads exceed the grid limit");
  SAGE_REQUIRE(heads_q % heads_kv == 0, "attn_fwd: num_qo_heads (%d) must be divisible by num_kv_heads (%d)", heads_q, heads_kv);
  SAGE_REQUIRE(granularity == SAGE_B200_GRAN_PER_THREAD || granularity == SAGE_B200_GRAN_PER_BLOCK,
               "attn_fwd: unknown granularity %d", granularity);
  SAGE_REQUIRE(pv_accum >= 0 && pv_accum <= 2, "attn_fwd: unknown pv_accum %d", pv_accum);
  if (head_dim != 64 && head_dim != 128) {
    if (head_dim == 256)
      return fail(SAGE_B200_ERR_UNSUPPORTED, "attn_fwd: head_dim 256 is not built yet");
    return fail(SAGE_B200_ERR_INVALID, "attn_fwd: head_dim must be 64 or 128 (pad first), got %d", head_dim);
  }
  SAGE_REQUIRE(blk_q == 32 || blk_q == 64 || blk_q == 128, "attn_fwd: blk_q must be 32, 64 or 128");
  if (blk_k != 64)
    return fail(SAGE_B200_ERR_UNSUPPORTED, "attn_fwd: only blk_k = 64 scale blocks are built (got %d)", blk_k);
  if (granularity == SAGE_B200_GRAN_PER_THREAD) {
    SAGE_REQUIRE(warp_q >= 8 && warp_q <= blk_q && (warp_q & (warp_q - 1)) == 0, "attn_fwd: bad warp_q %d", warp_q);
    if (warp_k != 64)
      return fail(SAGE_B200_ERR_UNSUPPORTED, "attn_fwd: only warp_k = 64 is built (got %d)", warp_k);
  }
  SAGE_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15u) == 0 && o_strides[0] % 8 == 0 && o_strides[1] % 8 == 0 &&
                   o_strides[2] % 8 == 0, "attn_fwd: output must be 16-byte aligned with strides % 8 == 0");

  AttnParams p;
  p.q_scale = q_scale;
  p.k_scale = k_scale;
  p.out = out;
  p.lse = lse;
  p.status = status;
  p.len_q = len_q;
  p.len_kv = len_kv;
  p.heads_q = heads_q;
  p.heads_kv = heads_kv;
  const int q_blocks = (len_q + blk_q - 1) / blk_q, k_blocks = (len_kv + blk_k - 1) / blk_k;
  if (granularity == SAGE_B200_GRAN_PER_THREAD) {
    p.q_groups = q_blocks * (blk_q / warp_q) * 8;
    p.k_groups = k_blocks * (blk_k / warp_k) * 4;
    p.warp_q = warp_q;
  } else {
    p.q_groups = q_blocks;
    p.k_groups = k_blocks;
    p.warp_q = blk_q;
  }
  p.gran = granularity;
  p.causal = is_causal ? 1 : 0;
  p.scale_log2 = sm_scale * kLog2e;
  p.os_b = o_strides[0];
  p.os_h = o_strides[1];
  p.os_n = o_strides[2];

  CUtensorMap mq, mk, mv;
  const CUtensorMapSwizzle swz_qk = (head_dim == 64) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  int rc = make_map(&mq, q, 1, batch, heads_q, len_q, head_dim, q_strides, head_dim, kTileQ, swz_qk, "q");
  if (rc) return rc;
  rc = make_map(&mk, k, 1, batch, heads_kv, len_kv, head_dim, k_strides, head_dim, kBlockKV, swz_qk, "k");
  if (rc) return rc;
  rc = make_map(&mv, v, 2, batch, heads_kv, len_kv, head_dim, v_strides, 64, kBlockKV, CU_TENSOR_MAP_SWIZZLE_128B, "v");
  if (rc) return rc;

  const dim3 grid((len_q + 2 * kTileQ - 1) / (2 * kTileQ), heads_q, batch);
  if (head_dim == 64) return launch_attn_mode<64>(pv_accum, out_dtype, mq, mk, mv, p, grid, stream);
  return launch_attn_mode<128>(pv_accum, out_dtype, mq, mk, mv, p, grid, stream);
}
