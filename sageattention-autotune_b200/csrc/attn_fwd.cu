// Host side of the attention core: argument checks, TMA tensor maps, kernel selection.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include "attn_common.cuh"
#include "attn_v1.cuh"
#include "attn_v4.cuh"
#include "attn_v5.cuh"
#include "tile_table.h"

namespace sage {

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

template <int D, int PV_MODE, int OUT_DTYPE, int KSUB>
static int launch_attn(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p,
                       cudaStream_t stream) {
  // Two kernels exist.  fp32, fp16 and fp8 accumulation run the two-tile kernel (attn_v1.cuh: up to 256 query
  // rows per CTA share every K/V block, the output accumulates in tensor memory).  The two-level
  // "fp16+fp32" mode needs an fp16 partial product next to the scores and runs the one-tile kernel with
  // a fold warpgroup (attn_v4.cuh) wherever the tile table says so; on the two-tile kernel it folds
  // inside the softmax warps.  KSUB = 2 (scale blocks of 32 keys, the reference's (128, 32, 32, 32)
  // candidate) is built into the two-tile kernel only.
  void (*kern)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const AttnParams) = nullptr;
  int smem = 0;
  int threads = kAttnThreads;
  int which = 0;               // index of the kernel in the per-device attribute cache below
  sage_b200_tile_entry te = tile_lookup(D, p.causal, PV_MODE, p.len_kv);
  // SAGE_B200_KERNEL=coupled overrides the table for sweeps and cross-checks: the two-level mode on the
  // two-tile kernel
  static const bool force_coupled = [] {
    const char* e = getenv("SAGE_B200_KERNEL");
    return e != nullptr && e[0] == 'c';
  }();
  if (force_coupled && te.kernel == SAGE_B200_KERNEL_ONE_TILE_FOLD) te.kernel = SAGE_B200_KERNEL_TWO_TILE_COUPLED;
  // SAGE_B200_KERNEL=persistent / =plain force the persistent or the one-CTA-per-tile form of the one-tile kernel
  static const int force_persistent = [] {
    const char* e = getenv("SAGE_B200_KERNEL");
    return (e != nullptr && e[0] == 'p' && e[1] == 'e') ? 1 : (e != nullptr && e[0] == 'p' && e[1] == 'l') ? 0 : -1;
  }();
  bool one_tile_fold = false, persistent = false;
  if constexpr (PV_MODE == SAGE_B200_PV_F16_F32 && D != 256 && KSUB == 1) {
    one_tile_fold = (te.kernel == SAGE_B200_KERNEL_ONE_TILE_FOLD || te.kernel == SAGE_B200_KERNEL_ONE_TILE_PERSISTENT);
    if (one_tile_fold) {
      persistent = force_persistent >= 0 ? force_persistent == 1 : te.kernel == SAGE_B200_KERNEL_ONE_TILE_PERSISTENT;
      if (persistent) {
        kern = v5::sage_attn_fwd_kernel<D, OUT_DTYPE>;
        smem = v5::SmemPlan<D>::kDynamic;
        which = 2;
      } else {
        kern = v4::sage_attn_fwd_kernel<D, OUT_DTYPE>;
        smem = v4::SmemPlan<D>::kDynamic;
        which = 1;
      }
      threads = v4::kThreads;
    }
  }
  constexpr bool kFp8 = (PV_MODE == SAGE_B200_PV_F8);
  if (!one_tile_fold) {
    kern = v1::sage_attn_fwd_kernel<D, PV_MODE, OUT_DTYPE, KSUB>;
    smem = v1::SmemPlan<D, kFp8>::kDynamic;
  }
  const int tiles = (one_tile_fold || D == 256) ? 1 : 2;
  const int rows_per_cta = tiles * kTileQ;
  dim3 grid((p.len_q + rows_per_cta - 1) / rows_per_cta, p.heads_q, p.batch);
  cudaError_t attr_err = cudaSuccess;
  // the attribute is per device: set it for every device that launches
  static bool done[3][64] = {};
  static int sm_count[64] = {};
  static std::mutex mu;
  int dev = 0;
  SAGE_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !done[which][dev]) {
      attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (attr_err != cudaSuccess)
        return fail(SAGE_B200_ERR_CUDA, "cudaFuncSetAttribute(%d bytes) failed: %s", smem, cudaGetErrorString(attr_err));
      if (dev >= 0 && dev < 64) done[which][dev] = true;
    }
  }
  if (persistent) {
    // one CTA per SM walks over the query tiles of all heads
    int sms = 0;
    {
      std::lock_guard<std::mutex> lock(mu);
      if (dev >= 0 && dev < 64 && sm_count[dev] == 0)
        SAGE_CUDA_TRY(cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
      sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 0;
    }
    if (sms <= 0) SAGE_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long items = static_cast<long long>(grid.x) * grid.y * grid.z;
    SAGE_REQUIRE(items < (1ll << 31), "attn_fwd: too many query tiles for one launch");
    grid = dim3(static_cast<unsigned>(items < sms ? items : sms), 1, 1);
  }
  SAGE_CUDA_TRY(launch_kernel(kern, grid, dim3(threads), smem, stream, mq, mk, mv, p));
  return SAGE_B200_OK;
}

template <int D, int PV_MODE, int KSUB>
static int launch_attn_out(int out_dtype, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                           const AttnParams& p, cudaStream_t stream) {
  if (out_dtype == SAGE_B200_BF16) return launch_attn<D, PV_MODE, SAGE_B200_BF16, KSUB>(mq, mk, mv, p, stream);
  return launch_attn<D, PV_MODE, SAGE_B200_F16, KSUB>(mq, mk, mv, p, stream);
}

template <int D, int KSUB>
static int launch_attn_mode(int pv_accum, int out_dtype, const CUtensorMap& mq, const CUtensorMap& mk,
                            const CUtensorMap& mv, const AttnParams& p, cudaStream_t stream) {
  switch (pv_accum) {
    case SAGE_B200_PV_F32: return launch_attn_out<D, SAGE_B200_PV_F32, KSUB>(out_dtype, mq, mk, mv, p, stream);
    case SAGE_B200_PV_F16: return launch_attn_out<D, SAGE_B200_PV_F16, KSUB>(out_dtype, mq, mk, mv, p, stream);
    case SAGE_B200_PV_F8: return launch_attn_out<D, SAGE_B200_PV_F8, KSUB>(out_dtype, mq, mk, mv, p, stream);
    default: return launch_attn_out<D, SAGE_B200_PV_F16_F32, KSUB>(out_dtype, mq, mk, mv, p, stream);
  }
}

}  // namespace sage

using namespace sage;

// budget of the kernels' bounded waits, in SM clocks (see sage_b200_set_wait_budget)
static std::atomic<long long> g_wait_cycles{kWaitCycles};

extern "C" long long sage_b200_set_wait_budget(long long cycles) {
  return g_wait_cycles.exchange(cycles > 0 ? cycles : kWaitCycles, std::memory_order_relaxed);
}

static int attn_fwd_impl(const int8_t* q, const int8_t* k, const void* v, const float* v_scale, const void* v_mean, void* out,
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
  SAGE_REQUIRE(pv_accum >= 0 && pv_accum <= 3, "attn_fwd: unknown pv_accum %d", pv_accum);
  SAGE_REQUIRE((pv_accum == SAGE_B200_PV_F8) == (v_scale != nullptr),
               "attn_fwd: the fp8 mode (and only it) takes a v_scale; use sage_b200_attn_fwd_fp8");
  SAGE_REQUIRE(v_scale == nullptr || aligned16(v_scale), "attn_fwd: v_scale must be 16-byte aligned");
  SAGE_REQUIRE(v_mean == nullptr || (pv_accum == SAGE_B200_PV_F16 && aligned16(v_mean)),
               "attn_fwd: a V mean goes with fp16 accumulation only and must be 16-byte aligned");
  SAGE_REQUIRE(granularity != SAGE_B200_GRAN_PER_THREAD || aligned16(k_scale),
               "attn_fwd: per-thread k_scale must be 16-byte aligned (it is read four groups at a time)");
  if (head_dim != 64 && head_dim != 128 && head_dim != 256)
    return fail(SAGE_B200_ERR_INVALID, "attn_fwd: head_dim must be 64, 128 or 256 (pad first), got %d", head_dim);
  SAGE_REQUIRE(blk_q == 16 || blk_q == 32 || blk_q == 64 || blk_q == 128, "attn_fwd: blk_q must be 16, 32, 64 or 128");
  SAGE_REQUIRE(blk_k == 64 || blk_k == 32, "attn_fwd: blk_k must be 64 or 32, got %d", blk_k);
  if (granularity == SAGE_B200_GRAN_PER_THREAD) {
    SAGE_REQUIRE(warp_q >= 8 && warp_q <= blk_q && (warp_q & (warp_q - 1)) == 0, "attn_fwd: bad warp_q %d", warp_q);
    if (warp_k != blk_k)
      return fail(SAGE_B200_ERR_UNSUPPORTED, "attn_fwd: only warp_k = blk_k is built (got %d, %d)", warp_k, blk_k);
  }
  SAGE_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15u) == 0 && o_strides[0] % 8 == 0 && o_strides[1] % 8 == 0 &&
                   o_strides[2] % 8 == 0, "attn_fwd: output must be 16-byte aligned with strides % 8 == 0");

  AttnParams p;
  p.q_scale = q_scale;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.v_mean = static_cast<const unsigned short*>(v_mean);
  p.out = out;
  p.lse = lse;
  p.status = status;
  static std::atomic<unsigned long long> next_launch_id{1};
  p.launch_id = next_launch_id.fetch_add(1, std::memory_order_relaxed);
  p.len_q = len_q;
  p.len_kv = len_kv;
  p.heads_q = heads_q;
  p.heads_kv = heads_kv;
  p.batch = batch;
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
  p.wait_cycles = g_wait_cycles.load(std::memory_order_relaxed);
  const PeerSet& peers = output_peers();
  p.n_peer = peers.n;
  for (int i = 0; i < kMaxPeers; ++i) p.peer_off[i] = i < peers.n ? peers.off[i] : 0;
  SAGE_REQUIRE(peers.n == 0 || ((reinterpret_cast<uintptr_t>(out) & 31u) == 0 && o_strides[0] % 16 == 0 &&
                                o_strides[1] % 16 == 0 && o_strides[2] % 16 == 0),
               "attn_fwd: with output peers the output must be 32-byte aligned with strides % 16 == 0");

  constexpr int kStageRows = 128;   // keys per TMA stage in both kernels
  CUtensorMap mq, mk, mv;
  const CUtensorMapSwizzle swz_qk = (head_dim == 64) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  const int box_qk = head_dim < 128 ? head_dim : 128;      // wider rows are staged as 128-byte panels
  int rc = make_map(&mq, q, 1, batch, heads_q, len_q, head_dim, q_strides, box_qk, kTileQ, swz_qk, "q");
  if (rc) return rc;
  rc = make_map(&mk, k, 1, batch, heads_kv, len_kv, head_dim, k_strides, box_qk, kStageRows, swz_qk, "k");
  if (rc) return rc;
  if (pv_accum == SAGE_B200_PV_F8)
    rc = make_map(&mv, v, 1, batch, heads_kv, len_kv, head_dim, v_strides, box_qk, kStageRows, swz_qk, "v");
  else
    rc = make_map(&mv, v, 2, batch, heads_kv, len_kv, head_dim, v_strides, 64, kStageRows, CU_TENSOR_MAP_SWIZZLE_128B, "v");
  if (rc) return rc;

  if (blk_k == 32) {
    if (head_dim == 64) return launch_attn_mode<64, 2>(pv_accum, out_dtype, mq, mk, mv, p, stream);
    if (head_dim == 256) return launch_attn_mode<256, 2>(pv_accum, out_dtype, mq, mk, mv, p, stream);
    return launch_attn_mode<128, 2>(pv_accum, out_dtype, mq, mk, mv, p, stream);
  }
  if (head_dim == 64) return launch_attn_mode<64, 1>(pv_accum, out_dtype, mq, mk, mv, p, stream);
  if (head_dim == 256) return launch_attn_mode<256, 1>(pv_accum, out_dtype, mq, mk, mv, p, stream);
  return launch_attn_mode<128, 1>(pv_accum, out_dtype, mq, mk, mv, p, stream);
}


extern "C" int sage_b200_tile_lookup(int head_dim, int is_causal, int pv_accum, int len_kv, sage_b200_tile_entry* entry) {
  SAGE_REQUIRE(entry != nullptr, "tile_lookup: null entry");
  SAGE_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "tile_lookup: head_dim must be 64, 128 or 256");
  SAGE_REQUIRE(pv_accum >= 0 && pv_accum <= 3 && len_kv > 0, "tile_lookup: bad pv_accum or length");
  *entry = tile_lookup(head_dim, is_causal, pv_accum, len_kv);
  return SAGE_B200_OK;
}

extern "C" int sage_b200_attn_fwd(const int8_t* q, const int8_t* k, const void* v, void* out,
                                  const float* q_scale, const float* k_scale, float* lse, int32_t* status,
                                  int out_dtype, int batch, int heads_q, int heads_kv, int len_q, int len_kv,
                                  int head_dim, const int64_t q_strides[3], const int64_t k_strides[3],
                                  const int64_t v_strides[3], const int64_t o_strides[3], int is_causal,
                                  float sm_scale, int blk_q, int blk_k, int warp_q, int warp_k,
                                  int granularity, int pv_accum, void* stream) {
  if (pv_accum == SAGE_B200_PV_F8)
    return fail(SAGE_B200_ERR_INVALID, "attn_fwd: the fp8 mode needs a v_scale; use sage_b200_attn_fwd_fp8");
  return attn_fwd_impl(q, k, v, nullptr, nullptr, out, q_scale, k_scale, lse, status, out_dtype, batch, heads_q, heads_kv,
                       len_q, len_kv, head_dim, q_strides, k_strides, v_strides, o_strides, is_causal, sm_scale,
                       blk_q, blk_k, warp_q, warp_k, granularity, pv_accum, stream);
}

extern "C" int sage_b200_attn_fwd_fuse_v_mean(const int8_t* q, const int8_t* k, const void* v, const void* v_mean,
                                              void* out, const float* q_scale, const float* k_scale, float* lse,
                                              int32_t* status, int out_dtype, int batch, int heads_q, int heads_kv,
                                              int len_q, int len_kv, int head_dim, const int64_t q_strides[3],
                                              const int64_t k_strides[3], const int64_t v_strides[3],
                                              const int64_t o_strides[3], int is_causal, float sm_scale, int blk_q,
                                              int blk_k, int warp_q, int warp_k, int granularity, void* stream) {
  SAGE_REQUIRE(v_mean != nullptr, "attn_fwd_fuse_v_mean: null v_mean");
  return attn_fwd_impl(q, k, v, nullptr, v_mean, out, q_scale, k_scale, lse, status, out_dtype, batch, heads_q,
                       heads_kv, len_q, len_kv, head_dim, q_strides, k_strides, v_strides, o_strides, is_causal,
                       sm_scale, blk_q, blk_k, warp_q, warp_k, granularity, SAGE_B200_PV_F16, stream);
}

extern "C" int sage_b200_attn_fwd_fp8(const int8_t* q, const int8_t* k, const void* v, const float* v_scale,
                                      void* out, const float* q_scale, const float* k_scale, float* lse,
                                      int32_t* status, int out_dtype, int batch, int heads_q, int heads_kv,
                                      int len_q, int len_kv, int head_dim, const int64_t q_strides[3],
                                      const int64_t k_strides[3], const int64_t v_strides[3],
                                      const int64_t o_strides[3], int is_causal, float sm_scale, int blk_q,
                                      int blk_k, int warp_q, int warp_k, int granularity, void* stream) {
  SAGE_REQUIRE(v_scale != nullptr, "attn_fwd_fp8: null v_scale");
  return attn_fwd_impl(q, k, v, v_scale, nullptr, out, q_scale, k_scale, lse, status, out_dtype, batch, heads_q, heads_kv,
                       len_q, len_kv, head_dim, q_strides, k_strides, v_strides, o_strides, is_causal, sm_scale,
                       blk_q, blk_k, warp_q, warp_k, granularity, SAGE_B200_PV_F8, stream);
}
