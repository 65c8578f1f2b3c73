// Output copies on other GPUs of the node: memory that the processes of the other GPUs can map, and the set
// of copies the attention launches of this thread write besides their own output.
//
// With heads sharded over the GPUs of a node (one process per GPU) every rank owns a slice of one output
// tensor.  When each rank needs the whole tensor, the attention epilogue stores every finished row into
// the same place of every other rank's tensor as well (plain stores to peer memory over NVLink), so the
// exchange rides along with the compute and no separate all-gather runs afterwards.
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace sage {

PeerSet& output_peers() {
  static thread_local PeerSet set;
  return set;
}

}  // namespace sage

using namespace sage;

static_assert(sizeof(cudaIpcMemHandle_t) == SAGE_B200_PEER_HANDLE_BYTES, "handle size");

// An interprocess handle names a whole driver allocation, and the process that opens it gets the address of
// that allocation's first byte.  The buffer is therefore only handed out when it starts its allocation
// (requests are rounded up to 2 MiB so that the driver does not carve them out of a shared block).
static bool starts_its_allocation(void* mem) {
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return false;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (reinterpret_cast<RangeFn>(sym)(&base, &size, reinterpret_cast<CUdeviceptr>(mem)) != CUDA_SUCCESS) return false;
  return base == reinterpret_cast<CUdeviceptr>(mem);
}

extern "C" int sage_b200_peer_alloc(size_t bytes, void** ptr, unsigned char* handle) {
  SAGE_REQUIRE(bytes > 0 && ptr != nullptr && handle != nullptr, "peer_alloc: null pointer or empty request");
  void* mem = nullptr;
  constexpr size_t kGrain = size_t(2) << 20;
  SAGE_CUDA_TRY(cudaMalloc(&mem, (bytes + kGrain - 1) / kGrain * kGrain));
  if (!starts_its_allocation(mem)) {
    cudaFree(mem);
    return fail(SAGE_B200_ERR_CUDA, "peer_alloc: the buffer does not start a driver allocation of its own");
  }
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, mem);
  if (e != cudaSuccess) {
    cudaFree(mem);
    return fail(SAGE_B200_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  std::memcpy(handle, &h, sizeof(h));
  *ptr = mem;
  return SAGE_B200_OK;
}

extern "C" int sage_b200_peer_open(const unsigned char* handle, void** ptr) {
  SAGE_REQUIRE(handle != nullptr && ptr != nullptr, "peer_open: null pointer");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  SAGE_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return SAGE_B200_OK;
}

extern "C" int sage_b200_peer_close(void* ptr) {
  SAGE_REQUIRE(ptr != nullptr, "peer_close: null pointer");
  SAGE_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return SAGE_B200_OK;
}

extern "C" int sage_b200_peer_free(void* ptr) {
  SAGE_REQUIRE(ptr != nullptr, "peer_free: null pointer");
  SAGE_CUDA_TRY(cudaFree(ptr));
  return SAGE_B200_OK;
}

extern "C" int sage_b200_set_output_peers(int n, const int64_t* byte_offsets) {
  SAGE_REQUIRE(n >= 0 && n <= kMaxOutputPeers, "set_output_peers: between 0 and %d peers, got %d", kMaxOutputPeers, n);
  SAGE_REQUIRE(n == 0 || byte_offsets != nullptr, "set_output_peers: null offsets");
  for (int i = 0; i < n; ++i)
    SAGE_REQUIRE(byte_offsets[i] != 0 && byte_offsets[i] % 32 == 0,
                 "set_output_peers: offset %d must be a non-zero multiple of 32 bytes", i);
  PeerSet& set = output_peers();
  set.n = n;
  for (int i = 0; i < n; ++i) set.off[i] = byte_offsets[i];
  return SAGE_B200_OK;
}
