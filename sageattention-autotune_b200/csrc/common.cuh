// Shared host/device helpers of the B200 SageAttention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/sage_b200.h"

namespace sage {

// Thread-local message behind sage_b200_last_error().
char* error_buffer();
int fail(int code, const char* fmt, ...);
// Every kernel launch of the library is counted (sage_b200_launch_count()).
void count_launch();

#define SAGE_CUDA_TRY(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return ::sage::fail(SAGE_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define SAGE_REQUIRE(cond, ...)                                           \
  do {                                                                    \
    if (!(cond)) return ::sage::fail(SAGE_B200_ERR_INVALID, __VA_ARGS__); \
  } while (0)

// Copies of the attention output in other GPUs' memory, for the launches of the calling thread
// (sage_b200_set_output_peers): byte offsets from the local output to each copy.
constexpr int kMaxOutputPeers = 7;
struct PeerSet {
  int n = 0;
  long long off[kMaxOutputPeers] = {};
};
PeerSet& output_peers();

// Programmatic dependent launch.  Inside one sage_b200_sageattn call the kernels form a chain on one
// stream; every kernel after the first is launched with the programmatic-serialisation attribute, so its
// CTAs may be placed (and run their set-up) while the previous kernel drains.  Each kernel of the
// library executes pdl_wait() before it touches global memory, which blocks until the previous kernel
// in the stream has completed and its writes are visible, and pdl_trigger() right at its start.  For a
// kernel launched the ordinary way both are no-ops.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// True while the calling thread is inside a chain whose next launch may overlap its predecessor.
bool& pdl_chain_flag();

struct PdlChain {            // RAII: the launches made while it lives, except the first, are dependent launches
  bool saved;
  PdlChain() : saved(pdl_chain_flag()) {}
  void arm() { pdl_chain_flag() = true; }
  ~PdlChain() { pdl_chain_flag() = saved; }
};

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_chain_flag() ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
  if (e == cudaSuccess) count_launch();
  return e;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// 16-bit storage -> fp32 (exact for both types).
template <int DTYPE>
__device__ __forceinline__ float to_f32(unsigned short bits) {
  if constexpr (DTYPE == SAGE_B200_BF16) {
    return __uint_as_float(static_cast<uint32_t>(bits) << 16);
  } else {
    return __half2float(__ushort_as_half(bits));
  }
}

template <int DTYPE>
__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (DTYPE == SAGE_B200_BF16) {
      x[2 * i + 0] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      x[2 * i + 0] = f.x;
      x[2 * i + 1] = f.y;
    }
  }
}

}  // namespace sage
