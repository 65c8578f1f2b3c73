// Thin inline-PTX wrappers for the sm_100a features the attention kernel uses:
// mbarrier, TMA tensor loads (no multicast), tcgen05 (TMEM alloc, MMA, commit, ld/st, fences),
// setmaxnreg, and the approximate math the reference kernel uses (ex2/lg2/rcp.approx.ftz,
// csrc/math.cuh:28-47 of the reference).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace sage {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " elect.sync _|p, 0xffffffff;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// non-blocking test of the same condition
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// the same with a suspend-time hint: the hardware may park the thread for up to `ns` nanoseconds
// (or until the phase completes) before the instruction returns
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}

// ------------------------------------------------------------------ TMA
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 4-D tiled load global -> shared of this CTA, completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// arrive on `bar` once every tcgen05 operation issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], int8 x int8 -> int32
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc], f16 x f16 -> f32 or f16
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc], e4m3 x e4m3 -> f32
__device__ __forceinline__ void mma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], f16 x f16
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base_lane + t)
#define SAGE_R32(a, o)                                                                                     \
  "=r"(a[o + 0]), "=r"(a[o + 1]), "=r"(a[o + 2]), "=r"(a[o + 3]), "=r"(a[o + 4]), "=r"(a[o + 5]),          \
      "=r"(a[o + 6]), "=r"(a[o + 7]), "=r"(a[o + 8]), "=r"(a[o + 9]), "=r"(a[o + 10]), "=r"(a[o + 11]),    \
      "=r"(a[o + 12]), "=r"(a[o + 13]), "=r"(a[o + 14]), "=r"(a[o + 15]), "=r"(a[o + 16]), "=r"(a[o + 17]), \
      "=r"(a[o + 18]), "=r"(a[o + 19]), "=r"(a[o + 20]), "=r"(a[o + 21]), "=r"(a[o + 22]), "=r"(a[o + 23]), \
      "=r"(a[o + 24]), "=r"(a[o + 25]), "=r"(a[o + 26]), "=r"(a[o + 27]), "=r"(a[o + 28]), "=r"(a[o + 29]), \
      "=r"(a[o + 30]), "=r"(a[o + 31])
#define SAGE_W32(a, o)                                                                                 \
  "r"(a[o + 0]), "r"(a[o + 1]), "r"(a[o + 2]), "r"(a[o + 3]), "r"(a[o + 4]), "r"(a[o + 5]),            \
      "r"(a[o + 6]), "r"(a[o + 7]), "r"(a[o + 8]), "r"(a[o + 9]), "r"(a[o + 10]), "r"(a[o + 11]),      \
      "r"(a[o + 12]), "r"(a[o + 13]), "r"(a[o + 14]), "r"(a[o + 15]), "r"(a[o + 16]), "r"(a[o + 17]),  \
      "r"(a[o + 18]), "r"(a[o + 19]), "r"(a[o + 20]), "r"(a[o + 21]), "r"(a[o + 22]), "r"(a[o + 23]),  \
      "r"(a[o + 24]), "r"(a[o + 25]), "r"(a[o + 26]), "r"(a[o + 27]), "r"(a[o + 28]), "r"(a[o + 29]),  \
      "r"(a[o + 30]), "r"(a[o + 31])

template <int OFF, int N>
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[N]) {
  static_assert(OFF + 32 <= N, "register window out of range");
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : SAGE_R32(r, OFF)
      : "r"(taddr)
      : "memory");
}
template <int OFF, int N>
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[N]) {
  static_assert(OFF + 32 <= N, "register window out of range");
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::SAGE_W32(r, OFF), "r"(taddr)
      : "memory");
}
// 16-column variants for roles that run on a small register budget
template <int OFF, int N>
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[N]) {
  static_assert(OFF + 16 <= N, "register window out of range");
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[OFF + 0]), "=r"(r[OFF + 1]), "=r"(r[OFF + 2]), "=r"(r[OFF + 3]), "=r"(r[OFF + 4]), "=r"(r[OFF + 5]),
        "=r"(r[OFF + 6]), "=r"(r[OFF + 7]), "=r"(r[OFF + 8]), "=r"(r[OFF + 9]), "=r"(r[OFF + 10]),
        "=r"(r[OFF + 11]), "=r"(r[OFF + 12]), "=r"(r[OFF + 13]), "=r"(r[OFF + 14]), "=r"(r[OFF + 15])
      : "r"(taddr)
      : "memory");
}
template <int OFF, int N>
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[N]) {
  static_assert(OFF + 16 <= N, "register window out of range");
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::"r"(r[OFF + 0]), "r"(r[OFF + 1]), "r"(r[OFF + 2]), "r"(r[OFF + 3]), "r"(r[OFF + 4]), "r"(r[OFF + 5]),
        "r"(r[OFF + 6]), "r"(r[OFF + 7]), "r"(r[OFF + 8]), "r"(r[OFF + 9]), "r"(r[OFF + 10]), "r"(r[OFF + 11]),
        "r"(r[OFF + 12]), "r"(r[OFF + 13]), "r"(r[OFF + 14]), "r"(r[OFF + 15]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ registers
template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ------------------------------------------------------------------ math
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// two fp32 -> packed fp16x2 (round to nearest even), `lo` in the low half
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// four fp32 -> packed e4m3x4 (round to nearest, saturating), v0 in the lowest byte
__device__ __forceinline__ uint32_t pack_e4m3x4(float v0, float v1, float v2, float v3) {
  uint32_t r;
  asm("{\n"
      " .reg .b16 lo, hi;\n"
      " cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n"
      " cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n"
      " mov.b32 %0, {lo, hi};\n"
      "}"
      : "=r"(r)
      : "f"(v0), "f"(v1), "f"(v2), "f"(v3));
  return r;
}
// fp32 accumulator + the fp16 value held in the low half of a 32-bit register, one instruction
// a (fp16, low half of `packed`) * b (fp16, low half of `b16`) + acc in one mixed-precision FMA
__device__ __forceinline__ float fma_f32_f16lo(uint32_t packed, uint32_t b16, float acc) {
  float r;
  asm("{\n"
      " .reg .b16 lo, hi, bl, bh;\n"
      " mov.b32 {lo, hi}, %1;\n"
      " mov.b32 {bl, bh}, %2;\n"
      " fma.rn.f32.f16 %0, lo, bl, %3;\n"
      "}"
      : "=f"(r)
      : "r"(packed), "r"(b16), "f"(acc));
  return r;
}
__device__ __forceinline__ float add_f32_f16lo(float acc, uint32_t packed) {
  float r;
  asm("{\n"
      " .reg .b16 lo, hi;\n"
      " mov.b32 {lo, hi}, %1;\n"
      " add.rn.f32.f16 %0, lo, %2;\n"
      "}"
      : "=f"(r)
      : "r"(packed), "f"(acc));
  return r;
}
// three-input maximum
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// packed pairs of fp32 (sm_100: one issue slot for two lanes)
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long sub2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// 2^y for a pair of arguments y <= 0 without the special-function unit (whose instructions hold the
// scheduler's dispatch port for most of their 8 cycles on this GPU): split y = n + f with n integer
// and f in [-0.5, 0.5] by a round-to-nearest add of 1.5*2^23, evaluate a degree-3 polynomial for
// 2^f (maximum relative error 7.5e-5, well under the 4.9e-4 rounding of the fp16 result), and add n
// to the exponent field.  Arguments below -126 are clamped; their results are far below fp16 range.
__device__ __forceinline__ void exp2_pair_poly(unsigned long long y2, float& p0, float& p1) {
  const unsigned long long magic = pack2(12582912.0f, 12582912.0f);
  const unsigned long long fr = add2(y2, magic);            // integer n in the low mantissa bits
  const unsigned long long f = add2(y2, sub2(magic, fr));   // y - n, exact
  unsigned long long q = fma2(pack2(0.055170975625514984f, 0.055170975625514984f), f,
                              pack2(0.24260970950126648f, 0.24260970950126648f));
  q = fma2(q, f, pack2(0.6932609677314758f, 0.6932609677314758f));
  q = fma2(q, f, pack2(0.9999281764030457f, 0.9999281764030457f));
  float q0, q1, r0, r1;
  unpack2(q, q0, q1);
  unpack2(fr, r0, r1);
  // n is clamped at -126 on its bit pattern (positive floats order like integers)
  const uint32_t n0 = max(__float_as_uint(r0), 0x4B400000u - 126u);
  const uint32_t n1 = max(__float_as_uint(r1), 0x4B400000u - 126u);
  p0 = __uint_as_float(__float_as_uint(q0) + (n0 << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (n1 << 23));
}

}  // namespace ptx
}  // namespace sage
