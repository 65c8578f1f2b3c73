// Shared pieces of the attention kernels: launch parameters, bounded mbarrier waits, the abort
// protocol and UMMA descriptors.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace sage {

constexpr int kTileQ = 128;
constexpr int kBlockKV = 128;
constexpr int kAttnThreads = 384;
constexpr int kKStages = 3;
constexpr int kVStages = 3;
constexpr long long kWaitCycles = 4000000000LL;   // default wait budget: about two seconds of SM clock
constexpr float kLog2e = 1.44269504088896340736f;
constexpr float kMagicF = 12582912.0f;            // 1.5 * 2^23
constexpr uint32_t kMagicI = 0x4B400000u;
constexpr float kLazyRescale = 8.0f;              // fp32 accumulators: rescale O only if max grew by 2^8

constexpr int kMaxPeers = kMaxOutputPeers;      // a node has at most eight GPUs

struct AttnParams {
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;          // fp8 P.V only: (batch, heads_kv, head_dim)
  const unsigned short* v_mean;  // fp16 accumulate with a smoothed V only: (batch, heads_kv, head_dim), output dtype
  void* out;
  float* lse;
  int32_t* status;
  int len_q, len_kv, heads_q, heads_kv, batch;
  int q_groups, k_groups;       // scale entries per head
  int warp_q;                    // WARPQ (per-thread) or BLKQ (per-block)
  int gran;
  int causal;
  float scale_log2;              // sm_scale * log2(e)
  int64_t os_b, os_h, os_n;
  unsigned long long launch_id;  // non-zero, unique per launch of this process (see g_attn_abort)
  long long wait_cycles;         // budget of every bounded wait, in SM clocks
  // Copies of the output in other GPUs' memory (head sharding with the exchange fused into the epilogue):
  // every row of the output is also stored at the same address plus peer_off[i], i < n_peer.  No fence
  // follows the stores: they are only read after the launch has completed (a system-scope fence per CTA
  // was measured and cost 6 % of a step for nothing).
  int n_peer;
  long long peer_off[kMaxPeers];
};

// The same 32 bytes (16 output values) to every peer copy of the output: plain stores that travel over
// NVLink, 32 bytes per store so that each request carries one whole sector.  `dst` is the address in the
// local output.
__device__ __forceinline__ void store_peers32(const AttnParams& p, const unsigned short* dst, const uint32_t* w) {
  for (int i = 0; i < p.n_peer; ++i) {
    const char* d = reinterpret_cast<const char*>(dst) + p.peer_off[i];
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(d), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
  }
}

// Abort protocol.  When a bounded wait runs out, the CTA records {launch id, wall time} in a device
// word pair; CTAs of the same launch that start later see it and return at once, so a launch whose
// pipeline is stuck ends after one wait period instead of one period per wave of CTAs, whether or not
// the caller passed a status word.  The record expires after kAbortHoldNs: a launch id that is baked
// into a captured graph is therefore not condemned for good, a later replay runs normally.
struct AbortRecord {
  unsigned long long id;
  unsigned long long when_ns;
};
static __device__ AbortRecord g_attn_abort = {0ull, 0ull};
constexpr unsigned long long kAbortHoldNs = 5000000000ull;

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool launch_aborted(const AttnParams& p) {
  const volatile AbortRecord* r = &g_attn_abort;
  if (r->id != p.launch_id) return false;
  return global_ns() - r->when_ns < kAbortHoldNs;
}
// `code` names the wait that ran out (or kCodeLateCta for a CTA that found the launch already aborted)
constexpr int kCodeLateCta = 99;
__device__ __forceinline__ void publish_abort(const AttnParams& p, int code) {
  if (code != kCodeLateCta) {
    volatile AbortRecord* r = &g_attn_abort;
    r->when_ns = global_ns();
    __threadfence();
    r->id = p.launch_id;
  }
  if (p.status != nullptr && atomicCAS_system(p.status, 0, code) == 0) {
    p.status[1] = blockIdx.x;
    p.status[2] = blockIdx.y;
    p.status[3] = blockIdx.z;
    __threadfence_system();
  }
}
// A CTA that gives up leaves no stale data behind: its rows of the output read as NaN.
__device__ __forceinline__ void poison_rows(const AttnParams& p, int rows, int q0, int b, int h, int head_dim) {
  for (int i = threadIdx.x; i < rows * (head_dim / 8); i += blockDim.x) {
    const int r = q0 + i / (head_dim / 8);
    if (r < p.len_q) {
      unsigned short* orow = static_cast<unsigned short*>(p.out) + b * p.os_b + h * p.os_h + r * p.os_n;
      const uint4 nan8 = make_uint4(0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu, 0x7fff7fffu);
      unsigned short* at = orow + (i % (head_dim / 8)) * 8;
      *reinterpret_cast<uint4*>(at) = nan8;
      for (int j = 0; j < p.n_peer; ++j) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(at) + p.peer_off[j]) = nan8;
    }
  }
}

// packed add of two values of the output type (reference: __hadd2 on DTypeOut2,
// csrc/qattn/qk_int8_sv_f16_kernel_sm80.cuh:551-569)
template <int OUT_DTYPE>
__device__ __forceinline__ uint32_t add2_out(uint32_t a, uint32_t b) {
  if constexpr (OUT_DTYPE == SAGE_B200_BF16) {
    const __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __half2 r = __hadd2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}

// Bounded mbarrier wait.  Returns false if the CTA is aborting.  A waiting thread should cost the
// scheduler little: after one non-blocking test the loop uses the form of try_wait that carries a
// suspend-time hint and looks at the abort flag and the clock between attempts.  (Measured on B200:
// the hint's value makes no difference, 0 / 2 / 20 us give the same kernel times, and a thinner loop that
// checks the flag and the clock only every 256 attempts runs the one-tile kernel 6 % slower.)
#ifndef SAGE_WAIT_HINT_NS
#define SAGE_WAIT_HINT_NS 2000
#endif
constexpr uint32_t kSuspendNs = SAGE_WAIT_HINT_NS;
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                         long long budget) {
  if (ptx::mbar_test_wait(bar, parity)) return true;       // the common case: the phase has completed
  const long long t0 = clock64();
  for (;;) {
    if (*abort_flag != 0) return false;
    if (clock64() - t0 > budget) {
      atomicCAS(const_cast<int*>(abort_flag), 0, code);
      return false;
    }
    if (kSuspendNs != 0 ? ptx::mbar_try_wait_suspend(bar, parity, kSuspendNs) : ptx::mbar_try_wait(bar, parity))
      return true;
  }
}

// Same, for code that goes on to warp-collective tcgen05.ld/st: the verdict is made warp-uniform.
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                              long long budget) {
  return __all_sync(0xffffffffu, wait_bar(bar, parity, abort_flag, code, budget));
}

// For the teardown of an aborting CTA: wait, with a fixed number of attempts, for a bulk copy that was
// already issued to land (its barrier phase to complete).  Shared memory must not receive data after
// the CTA has exited.
__device__ __forceinline__ bool drain_bar(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < 200000; ++i)
    if (ptx::mbar_try_wait_suspend(bar, parity, 1000u)) return true;
  return false;
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

// fp8 P.V: e4m3 x e4m3 -> fp32, A from tensor memory, B MN-major, M = 128, N = D
template <int D>
__host__ __device__ constexpr uint32_t idesc_pv_f8() {
  return (1u << 4) | (0u << 7) | (0u << 10) | (1u << 16) | ((uint32_t(D) >> 3) << 17) | ((kTileQ >> 4) << 24);
}
// MN-major fp8 operand: V as [keys][D bytes], D = 128 -> 128-byte swizzle, D = 64 -> 64-byte swizzle
template <int D>
__device__ __forceinline__ uint64_t desc_mnmajor_f8(uint32_t smem_addr) {
  constexpr uint64_t layout = (D == 128) ? 2 : 4;
  constexpr uint64_t sbo = (8 * D) >> 4;                     // 8 keys
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (sbo << 32) |
         (uint64_t(1) << 46) | (layout << 61);
}
constexpr float kLog2Of448 = 8.807354922057604f;             // P is scaled by 448 before rounding to e4m3

template <int OUT_DTYPE>
__device__ __forceinline__ uint32_t pack_out(float lo, float hi) {
  if constexpr (OUT_DTYPE == SAGE_B200_BF16) return ptx::pack_bf16x2(lo, hi);
  else return ptx::pack_f16x2(lo, hi);
}


}  // namespace sage
