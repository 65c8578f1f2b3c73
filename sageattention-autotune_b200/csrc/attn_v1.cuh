// Two-tile kernel of the SageAttention core for B200 (sm_100a): int8 Q.K^T and fp16 (or fp8) P.V on tcgen05 tensor cores with
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
#pragma once

#include "attn_common.cuh"

namespace sage {
namespace v1 {

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

// head_dim 256 runs this kernel with ONE query tile per CTA (S + a 256-column O fill tensor memory
// for one tile only) and two K/V stages instead of three (Q 32 KB + 2 x 32 KB + 2 x 64 KB = 224 KB).
// (One tile per CTA for the smaller head dims as well was measured and dropped: twice the CTAs, but each
// K/V block fetched per 128 instead of 256 query rows; 20-60 % slower from N = 1024 to 16384, causal or not.)
template <int D, bool F8 = false>
struct SmemPlan {
  static constexpr int kTiles = (D == 256) ? 1 : 2;
  static constexpr int kStagesK = (D == 256) ? 2 : kKStages;
  static constexpr int kStagesV = (D == 256) ? 2 : kVStages;
  static constexpr int kQBytes = kTileQ * D;                 // int8
  static constexpr int kKBytes = kBlockKV * D;               // int8
  static constexpr int kVBytes = kBlockKV * D * (F8 ? 1 : 2);  // fp16, or e4m3
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kTiles * kQBytes;
  static constexpr int kVOff = kKOff + kStagesK * kKBytes;
  static constexpr int kBarOff = kVOff + kStagesV * kVBytes;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;             // slack for manual 1024-byte alignment
};


// Scale class of column c of a 128-key block.  KSUB = 64 / BLKK scale blocks per 64 keys: the reference's
// candidates use BLKK = WARPK = 64 (eight classes per block) or 32 (sixteen).
template <int KSUB>
__device__ __forceinline__ constexpr int k_class(int c) { return ((c / (64 / KSUB)) << 2) | ((c & 7) >> 1); }

// One softmax warpgroup: thread `row` (0..127) of tile `tile`.
template <int D, int PV_MODE, int OUT_DTYPE, int KSUB>
__device__ __forceinline__ void softmax_role(const AttnParams& p, uint32_t bars, uint32_t tmem_base,
                                             volatile int* abort_flag, int tile, int row, int n_blocks,
                                             int q_row0, int b, int h, int h_kv) {
  constexpr bool kF16Acc = (PV_MODE == SAGE_B200_PV_F16);
  constexpr bool kInstBuf = (PV_MODE == SAGE_B200_PV_F16_F32);
  constexpr bool kFp8 = (PV_MODE == SAGE_B200_PV_F8);
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
  // scales of block j: four per scale block of 64 / KSUB keys in the per-thread layout (vector loads),
  // one per scale block in the per-block layout (replicated over the four classes)
  constexpr int kNA = 8 * KSUB;
  const bool per_thread = (p.gran == SAGE_B200_GRAN_PER_THREAD);
  auto load_scales = [&](int j, float (&a)[kNA]) {
#pragma unroll
    for (int u = 0; u < 2 * KSUB; ++u) {
      float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
      if (per_thread) {
        if (j * kNA + 4 * u + 3 < p.k_groups)
          asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(f.x), "=f"(f.y), "=f"(f.z), "=f"(f.w) : "l"(ks_base + kNA * j + 4 * u));
      } else if (2 * KSUB * j + u < p.k_groups) {
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(f.x) : "l"(ks_base + 2 * KSUB * j + u));
        f.y = f.z = f.w = f.x;
      }
      a[4 * u + 0] = f.x, a[4 * u + 1] = f.y, a[4 * u + 2] = f.z, a[4 * u + 3] = f.w;
    }
  };

#pragma unroll 1
  for (int j = 0; j < n_blocks; ++j) {
    const int k0 = j * kBlockKV;
    // the 8 * KSUB dequantisation constants of this block; the next block's line is pulled into L1 now
    // so that its loads do not pay an L2 round trip (registers are too scarce to hold them a block ahead)
    float a[kNA];
    load_scales(j, a);
    if (j + 1 < n_blocks)
      asm volatile("prefetch.global.L1 [%0];" ::"l"(ks_base + (per_thread ? kNA : 2 * KSUB) * (j + 1)));
#pragma unroll
    for (int t = 0; t < kNA; ++t) a[t] = p.scale_log2 * (q_sc * a[t]);

    ok = wait_bar_warp(bar_s_full, j & 1, abort_flag, 10 + tile, p.wait_cycles);
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
      // X = float(S) + 1.5*2^23 without a conversion: |S| < 2^22, so adding S to the bit pattern of
      // 1.5*2^23 is exact.  X is monotonic in S, so the row maximum is taken on X (three-input max),
      // per scale class, and mapped back through the class's constants.
#pragma unroll
      for (int c = 0; c < 128; ++c) s[c] += kMagicI;
#pragma unroll
      for (int t = 0; t < kNA; ++t) {
        constexpr int kSpan = 64 / KSUB;                    // keys per scale block
        constexpr int kVals = kSpan / 4;                    // columns of one class in it
        const int base = (t >> 2) * kSpan + (t & 3) * 2;    // the class owns columns base + 8i, base + 8i + 1
        float v[kVals];
#pragma unroll
        for (int i = 0; i < kVals / 2; ++i) {
          v[2 * i] = __uint_as_float(s[base + 8 * i]);
          v[2 * i + 1] = __uint_as_float(s[base + 8 * i + 1]);
        }
        float mx = v[0];
#pragma unroll
        for (int i = 1; i < kVals - 1; i += 2) mx = ptx::max3(mx, v[i], v[i + 1]);
        mx = fmaxf(mx, v[kVals - 1]);
        m_blk = fmaxf(m_blk, (mx - kMagicF) * a[t]);
      }
    } else {
      // diagonal or ragged block: scale first, mask to -inf, keep the scaled values in place
      const int lim_causal = p.causal ? (q_row - k0) : kBlockKV;     // columns <= lim are visible
      const int lim_len = p.len_kv - k0 - 1;
      const int lim = min(lim_causal, lim_len);
#pragma unroll
      for (int c = 0; c < 128; ++c) {
        float x = static_cast<float>(static_cast<int>(s[c])) * a[k_class<KSUB>(c)];
        x = (c <= lim) ? x : -INFINITY;
        m_blk = fmaxf(m_blk, x);
        s[c] = __float_as_uint(x);
      }
    }
    m_run = fmaxf(m_run, m_blk);

    // Choose the reference point and the factor by which earlier work must shrink.  fp32 accumulators
    // tolerate P up to 2^8 and move the reference lazily.  The fp16 accumulators need P <= 1; their
    // reference is the running maximum rounded UP to a multiple of 4, which still bounds P by 1 (the
    // largest P of a row is at least 2^-4: no loss of fp16 precision), moves only when the maximum
    // crosses such a multiple (rarely after the first blocks, so the rescale of O is skipped for most
    // blocks) and makes every rescale factor an exact power of two.  The e4m3 P keeps
    // the exact maximum: with three mantissa bits the rounding pattern of P depends on the reference,
    // and the published scheme (and its CPU emulation) rounds 448 * 2^(s - max).
    constexpr bool kIntRef = kF16Acc || kInstBuf;
    constexpr bool kTightRef = kIntRef || kFp8;
    float alpha = 1.0f;
    bool rescale = false;
    if (j == 0) {
      m_used = kIntRef ? ceilf(m_run * 0.25f) * 4.0f : m_run;
    } else {
      const float grow = m_run - m_used;
      if (kTightRef ? (grow > 0.0f) : (grow > kLazyRescale)) {
        const float m_next = kIntRef ? ceilf(m_run * 0.25f) * 4.0f : m_run;
        if constexpr (kIntRef) {
          // 2^(m_used - m_next) for integer arguments, exactly; 0 below the normal range
          const int e = static_cast<int>(fmaxf(m_used - m_next, -127.0f)) + 127;
          alpha = __int_as_float(e << 23);
        } else {
          alpha = ptx::ex2(m_used - m_next);
        }
        m_used = m_next;
        rescale = true;
      }
    }
    // a row that has seen nothing visible yet keeps a finite reference so that 2^(-inf - m) = 0
    const float m_ref = ((m_used == -INFINITY) ? 0.0f : m_used) - (kFp8 ? kLog2Of448 : 0.0f);

    if constexpr (!kInstBuf) {
      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
        ok = wait_bar_warp(bar_pv_done, (j - 1) & 1, abort_flag, 20 + tile, p.wait_cycles);
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
    // Of every kPolyDen groups of four columns, kPolyNum evaluate 2^x with a polynomial on the FMA pipe
    // and the rest with ex2.approx on the special-function unit, so that both pipes work: measured
    // at N = 32768 the fp32 mode takes 14.6 ms with 0/8, 12.95 ms with 3/8, 13.8 ms with 4/8, 19 ms with
    // 8/8 (first launches; once the 1000 W power cap lowers the clock: 15.3 / 14.7 ms with 0/8 / 3/8);
    // the fp16+fp32 mode of this kernel is bound by its hand-over chain and is indifferent (2/8 kept).
    constexpr int kPolyDen = 8;
#ifndef SAGE_V1_POLY
#define SAGE_V1_POLY 3
#endif
    constexpr int kPolyNum = kInstBuf ? 2 : SAGE_V1_POLY;
    if (!need_mask) {
      // p = 2^(X*a + neg) with neg = -(1.5*2^23*a + m); two columns of one class per packed FMA
      // (with sixteen classes the packed constants are built per scale block of 32 keys: holding all of
      // them would cost 64 registers)
      constexpr int kHeld = (KSUB == 1) ? 8 : 4;
      unsigned long long a2[kHeld], neg2[kHeld];
      if constexpr (KSUB == 1) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float ng = fmaf(-kMagicF, a[t], -m_ref);
          a2[t] = ptx::pack2(a[t], a[t]);
          neg2[t] = ptx::pack2(ng, ng);
        }
      }
      unsigned long long acc0 = ptx::pack2(0.0f, 0.0f), acc1 = acc0;
#pragma unroll
      for (int c = 0; c < 128; c += 4) {
        if constexpr (KSUB == 2) {
          if ((c & 31) == 0) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float at = a[(c >> 5) * 4 + t];
              const float ng = fmaf(-kMagicF, at, -m_ref);
              a2[t] = ptx::pack2(at, at);
              neg2[t] = ptx::pack2(ng, ng);
            }
          }
        }
        constexpr int kMask = (KSUB == 1) ? 7 : 3;          // index into the constants that are held
        const unsigned long long e0 = ptx::fma2(ptx::pack2(__uint_as_float(s[c + 0]), __uint_as_float(s[c + 1])),
                                                a2[k_class<KSUB>(c) & kMask], neg2[k_class<KSUB>(c) & kMask]);
        const unsigned long long e1 = ptx::fma2(ptx::pack2(__uint_as_float(s[c + 2]), __uint_as_float(s[c + 3])),
                                                a2[k_class<KSUB>(c + 2) & kMask], neg2[k_class<KSUB>(c + 2) & kMask]);
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
        if constexpr (kFp8) {
          s[c / 4] = ptx::pack_e4m3x4(p0, p1, p2, p3);
        } else {
          s[c / 2 + 0] = ptx::pack_f16x2(p0, p1);
          s[c / 2 + 1] = ptx::pack_f16x2(p2, p3);
        }
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
        if constexpr (kFp8) {
          s[c / 4] = ptx::pack_e4m3x4(p0, p1, p2, p3);
        } else {
          s[c / 2 + 0] = ptx::pack_f16x2(p0, p1);
          s[c / 2 + 1] = ptx::pack_f16x2(p2, p3);
        }
      }
    }
    d_sum = d_sum * alpha + ((sum0 + sum1) + (sum2 + sum3));

    ptx::tmem_st32<0>(t_p + 0, s);
    if constexpr (!kFp8) ptx::tmem_st32<32>(t_p + 32, s);     // e4m3: four keys per column, 32 columns
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
    ptx::mbar_arrive(bar_p_full);

    if constexpr (kInstBuf) {
      // "fp16+fp32": this block's P.V is accumulated in fp16 from zero, 64 channels at a time, and
      // folded into the fp32 O (compute_fp16_sv_permuted_inst_buf, attn_utils.cuh:447-518)
      const bool any_rescale = __any_sync(0xffffffffu, rescale);
#pragma unroll 1
      for (int ch = 0; ch < D / 64 && ok; ++ch) {
        ok = wait_bar_warp(bar_pv_done, (j * (D / 64) + ch) & 1, abort_flag, 30 + tile, p.wait_cycles);
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
            o[i] = __float_as_uint(ptx::add_f32_f16lo(acc, t16[i]));
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
      ok = wait_bar_warp(bar_pv_done, (n_blocks - 1) & 1, abort_flag, 40 + tile, p.wait_cycles);
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
        if (p.v_mean != nullptr) {
          // V was smoothed by its channel mean: add the mean back, in the output type
          const uint4* vm = reinterpret_cast<const uint4*>(p.v_mean + (static_cast<int64_t>(b) * p.heads_kv + h_kv) * D + c0);
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            const uint4 m4 = __ldg(vm + i / 4);
            w[i] = add2_out<OUT_DTYPE>(w[i], m4.x);
            w[i + 1] = add2_out<OUT_DTYPE>(w[i + 1], m4.y);
            w[i + 2] = add2_out<OUT_DTYPE>(w[i + 2], m4.z);
            w[i + 3] = add2_out<OUT_DTYPE>(w[i + 3], m4.w);
          }
        }
        if (store) {
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<uint4*>(orow + c0 + 2 * i) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
          store_peers32(p, orow + c0, w);
          store_peers32(p, orow + c0 + 16, w + 8);
        }
      }
    } else {
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t o[32];
        ptx::tmem_ld32<0>(t_o + c0, o);
        ptx::tmem_wait_ld();
        uint32_t w[16];
        if constexpr (kFp8) {
          const float4* vs = reinterpret_cast<const float4*>(
              p.v_scale + (static_cast<int64_t>(b) * p.heads_kv + h_kv) * D + c0);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 sc = __ldg(vs + i);
            w[2 * i] = pack_out<OUT_DTYPE>(__uint_as_float(o[4 * i]) * inv * sc.x, __uint_as_float(o[4 * i + 1]) * inv * sc.y);
            w[2 * i + 1] = pack_out<OUT_DTYPE>(__uint_as_float(o[4 * i + 2]) * inv * sc.z, __uint_as_float(o[4 * i + 3]) * inv * sc.w);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            w[i] = pack_out<OUT_DTYPE>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
        }
        if (store) {
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<uint4*>(orow + c0 + 2 * i) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
          store_peers32(p, orow + c0, w);
          store_peers32(p, orow + c0 + 16, w + 8);
        }
      }
    }
    if (p.lse != nullptr && store)
      p.lse[(static_cast<int64_t>(b) * p.heads_q + h) * p.len_q + q_row] =
          ptx::lg2(d_sum) + m_used - (kFp8 ? kLog2Of448 : 0.0f);
  }
  ptx::tc_fence_before();
}

template <int D, int PV_MODE, int OUT_DTYPE, int KSUB = 1>
__global__ void __launch_bounds__(kAttnThreads, 1)
sage_attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  constexpr bool kFp8 = (PV_MODE == SAGE_B200_PV_F8);
  using Plan = SmemPlan<D, kFp8>;
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
  constexpr int kTiles = Plan::kTiles;
  constexpr int kStK = Plan::kStagesK, kStV = Plan::kStagesV;
  const int pair = p.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int q0 = pair * kTiles * kTileQ;

  int n_blk[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = q0 + t * kTileQ;
    int kv_end = p.causal ? min(p.len_kv, r0 + kTileQ) : p.len_kv;
    n_blk[t] = (t < kTiles && r0 < p.len_q) ? (kv_end + kBlockKV - 1) / kBlockKV : 0;
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
    // another CTA of this launch already gave up: do not queue more bounded waits behind it.  One thread
    // decides for the whole CTA, and every thread reads the verdict after the barrier below.
    *abort_flag = launch_aborted(p) ? kCodeLateCta : 0;
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
  // the set-up above touched no global memory; what follows reads what the previous kernel wrote
  pdl_trigger();
  pdl_wait();
  const bool late = (*abort_flag != 0);

  if (late) {
    // nothing was issued: fall through to the teardown
  } else if (warp < 8) {
    ptx::reg_inc<232>();
    const int tile = warp >> 2;
    softmax_role<D, PV_MODE, OUT_DTYPE, KSUB>(p, bars, tmem_base, abort_flag, tile, threadIdx.x & 127, n_blk[tile],
                                        q0 + tile * kTileQ, b, h, h_kv);
  } else {
    ptx::reg_dec<40>();
    if (warp == 8 && lane == 0) {
      // ---------------- TMA producer ----------------
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      const uint32_t q_smem = smem_base + Plan::kQOff;
      // Q and K rows wider than one 128-byte swizzle span (head_dim 256) are staged as panels of 128 bytes
      constexpr int kPanelBytesQK = (D == 64) ? 64 : 128;
      constexpr int kPanelsQKLoad = D / kPanelBytesQK;
      ptx::mbar_arrive_expect_tx(bars + 8 * kBarQFull, kTiles * Plan::kQBytes);
#pragma unroll
      for (int t = 0; t < kTiles; ++t)
#pragma unroll
        for (int pn = 0; pn < kPanelsQKLoad; ++pn)
          ptx::tma_load_4d(q_smem + t * Plan::kQBytes + pn * (kTileQ * kPanelBytesQK), &tm_q, bars + 8 * kBarQFull,
                           pn * kPanelBytesQK, q0 + t * kTileQ, h, b);
      bool ok = true;
      int j_k = 0, j_v = 0;      // blocks whose K / V copy was issued
#pragma unroll 1
      for (int j = 0; j < n_max && ok; ++j) {
        const int ks = j % kStK, vs = j % kStV;
        ok = wait_bar(bars + 8 * (kBarKEmpty + ks), ((j / kStK) & 1) ^ 1, abort_flag, 50, p.wait_cycles);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bars + 8 * (kBarKFull + ks), Plan::kKBytes);
#pragma unroll
        for (int pn = 0; pn < kPanelsQKLoad; ++pn)
          ptx::tma_load_4d(smem_base + Plan::kKOff + ks * Plan::kKBytes + pn * (kBlockKV * kPanelBytesQK), &tm_k,
                           bars + 8 * (kBarKFull + ks), pn * kPanelBytesQK, j * kBlockKV, h_kv, b);
        j_k = j + 1;
        ok = wait_bar(bars + 8 * (kBarVEmpty + vs), ((j / kStV) & 1) ^ 1, abort_flag, 51, p.wait_cycles);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(bars + 8 * (kBarVFull + vs), Plan::kVBytes);
#pragma unroll
        // fp16: 64-channel panels; e4m3: panels of up to 128 channels; either way 128 bytes per key and panel
        for (int pn = 0; pn < (kFp8 ? (D > 128 ? D / 128 : 1) : D / 64); ++pn)
          ptx::tma_load_4d(smem_base + Plan::kVOff + vs * Plan::kVBytes + pn * (kBlockKV * 128), &tm_v,
                           bars + 8 * (kBarVFull + vs), pn * (kFp8 ? 128 : 64), j * kBlockKV, h_kv, b);
        j_v = j + 1;
      }
      // Leave no copy in flight behind us, whatever made the roles stop: wait (bounded) for Q and for the
      // copies of the last stages' worth of blocks (earlier ones had landed before their stage was handed
      // back).  After a normal run these phases completed long ago and every wait returns at once.
      drain_bar(bars + 8 * kBarQFull, 0);
      for (int j = max(0, j_k - kStK); j < j_k; ++j) drain_bar(bars + 8 * (kBarKFull + j % kStK), (j / kStK) & 1);
      for (int j = max(0, j_v - kStV); j < j_v; ++j) drain_bar(bars + 8 * (kBarVFull + j % kStV), (j / kStV) & 1);
    } else if (warp == 9) {
      // ---------------- MMA issuer ----------------
      // The whole warp runs this loop and one elected lane issues: operands that are computed in
      // converged code stay in uniform registers, which tcgen05.mma and tcgen05.commit read directly.
      auto commit = [&](uint32_t bar) {
        if (ptx::elect_one()) ptx::tc_commit(bar);
        __syncwarp();
      };
      constexpr int kRowBytesQK = (D == 64) ? 64 : 128;
      constexpr int kPanelsQK = D / kRowBytesQK;              // 1 (2 for D = 256)
      constexpr int kStepsPerPanel = kRowBytesQK / 32;        // int8: 32 bytes of K per instruction
      const uint32_t q_smem = smem_base + Plan::kQOff;
      const uint32_t k_smem = smem_base + Plan::kKOff;
      const uint32_t v_smem = smem_base + Plan::kVOff;
      const uint32_t idq = idesc_qk();
      const uint32_t idp = kFp8 ? idesc_pv_f8<D>() : idesc_pv<D, kF16Acc>();
      const uint32_t idp_chunk = idesc_pv<64, true>();

      // Descriptors differ only in their 14-bit start-address field (units of 16 bytes), which never
      // carries out of the field for shared-memory addresses: build them once, then add offsets.
      const uint64_t q_desc0 = desc_kmajor<kRowBytesQK>(q_smem);
      const uint64_t k_desc0 = desc_kmajor<kRowBytesQK>(k_smem);
      const uint64_t v_desc0 = (kFp8 && D <= 128) ? desc_mnmajor_f8<(D <= 128 ? D : 128)>(v_smem)
                                                  : desc_mnmajor(v_smem, kBlockKV * 128);

      auto issue_qk = [&](int t, int stage) {
        const uint32_t d_t = tmem_base + t * 256;
        const uint64_t da0 = q_desc0 + static_cast<uint64_t>((t * Plan::kQBytes) >> 4);
        const uint64_t db0 = k_desc0 + static_cast<uint64_t>((stage * Plan::kKBytes) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int pn = 0; pn < kPanelsQK; ++pn) {
#pragma unroll
            for (int s = 0; s < kStepsPerPanel; ++s) {
              const uint64_t off = static_cast<uint64_t>((pn * (kTileQ * kRowBytesQK) + s * 32) >> 4);
              ptx::mma_i8_ss(d_t, da0 + off, db0 + off, idq, (pn | s) != 0);
            }
          }
        }
        __syncwarp();
      };
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t d_t = tmem_base + t * 256 + 128;
        const uint32_t a_t = tmem_base + t * 256;
        const uint64_t db0 = v_desc0 + static_cast<uint64_t>((stage * Plan::kVBytes) >> 4);
        if (ptx::elect_one()) {
          if constexpr (kFp8) {
#pragma unroll
            for (int s = 0; s < kBlockKV / 32; ++s)   // 32 keys per instruction: 8 columns of P, 32 rows of V
              ptx::mma_f8_ts(d_t, a_t + s * 8, db0 + static_cast<uint64_t>((s * 32 * (D > 128 ? 128 : D)) >> 4), idp,
                             (accumulate || s != 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int s = 0; s < kBlockKV / 16; ++s) {
              // 16 keys per instruction: 8 packed columns of P, 16 rows (2 KB) of every V panel
              ptx::mma_f16_ts(d_t, a_t + s * 8, db0 + static_cast<uint64_t>((s * 2048) >> 4), idp,
                              (accumulate || s != 0) ? 1u : 0u);
            }
          }
        }
        __syncwarp();
      };
      // "fp16+fp32": one 64-channel panel of V at a time into the fp16 scratch columns
      auto issue_pv_chunk = [&](int t, int stage, int ch) {
        const uint32_t d_t = tmem_base + t * 256 + 64;
        const uint32_t a_t = tmem_base + t * 256;
        const uint64_t db0 = v_desc0 + static_cast<uint64_t>((stage * Plan::kVBytes + ch * (kBlockKV * 128)) >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int s = 0; s < kBlockKV / 16; ++s)
            ptx::mma_f16_ts(d_t, a_t + s * 8, db0 + static_cast<uint64_t>((s * 2048) >> 4), idp_chunk, s != 0 ? 1u : 0u);
        }
        __syncwarp();
      };

      bool ok = wait_bar_warp(bars + 8 * kBarQFull, 0, abort_flag, 60, p.wait_cycles);
      if (ok && n_max > 0) ok = wait_bar_warp(bars + 8 * (kBarKFull + 0), 0, abort_flag, 61, p.wait_cycles);
      if (ok && n_max > 0) {
        ptx::tc_fence_after();
        for (int t = 0; t < 2; ++t) {
          if (n_blk[t] > 0) {
            issue_qk(t, 0);
            commit(bars + 8 * (kBarSFull + t));
          }
        }
        commit(bars + 8 * (kBarKEmpty + 0));
      }
#pragma unroll 1
      for (int j = 0; j < n_max && ok; ++j) {
        const int vs = j % kStV;
        const int nxt = j + 1;
        const int ks = nxt % kStK;
        ok = wait_bar_warp(bars + 8 * (kBarVFull + vs), (j / kStV) & 1, abort_flag, 62, p.wait_cycles);
        if (!ok) break;
        if (nxt < n_max) {
          ok = wait_bar_warp(bars + 8 * (kBarKFull + ks), (nxt / kStK) & 1, abort_flag, 63, p.wait_cycles);
          if (!ok) break;
        }
        if constexpr (!kInstBuf) {
          for (int t = 0; t < 2 && ok; ++t) {
            if (j < n_blk[t]) {
              ok = wait_bar_warp(bars + 8 * (kBarPFull + t), j & 1, abort_flag, 64 + t, p.wait_cycles);
              if (!ok) break;
              ptx::tc_fence_after();
              issue_pv(t, vs, j > 0);
              commit(bars + 8 * (kBarPvDone + t));
              if (nxt < n_blk[t]) {
                issue_qk(t, ks);
                commit(bars + 8 * (kBarSFull + t));
              }
            }
          }
        } else {
          constexpr int kChunks = D / 64;
          for (int ch = 0; ch < kChunks && ok; ++ch) {
            for (int t = 0; t < 2 && ok; ++t) {
              if (j < n_blk[t]) {
                if (ch == 0) ok = wait_bar_warp(bars + 8 * (kBarPFull + t), j & 1, abort_flag, 64 + t, p.wait_cycles);
                else ok = wait_bar_warp(bars + 8 * (kBarSFree + t), (j * kChunks + ch - 1) & 1, abort_flag, 66 + t, p.wait_cycles);
                if (!ok) break;
                ptx::tc_fence_after();
                issue_pv_chunk(t, vs, ch);
                commit(bars + 8 * (kBarPvDone + t));
              }
            }
          }
          for (int t = 0; t < 2 && ok; ++t) {
            if (nxt < n_blk[t]) {
              ok = wait_bar_warp(bars + 8 * (kBarSFree + t), (j * kChunks + kChunks - 1) & 1, abort_flag, 68 + t, p.wait_cycles);
              if (!ok) break;
              ptx::tc_fence_after();
              issue_qk(t, ks);
              commit(bars + 8 * (kBarSFull + t));
            }
          }
        }
        if (!ok) break;
        commit(bars + 8 * (kBarVEmpty + vs));
        if (nxt < n_max) commit(bars + 8 * (kBarKEmpty + ks));
      }
      // everything this thread issued must have retired before tensor memory is released
      commit(bars + 8 * kBarDrain);
      for (int i = 0; i < (1 << 20) && !ptx::mbar_try_wait(bars + 8 * kBarDrain, 0); ++i) {}
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (warp == 8) ptx::tmem_dealloc(tmem_base, 512);
  if (*abort_flag != 0) {
    poison_rows(p, kTiles * kTileQ, q0, b, h, D);
    if (threadIdx.x == 0) publish_abort(p, *abort_flag);
  }
}


}  // namespace v1
}  // namespace sage
