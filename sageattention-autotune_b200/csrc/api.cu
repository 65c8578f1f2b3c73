// Error reporting and version entry points of the C ABI.
#include <atomic>

#include "common.cuh"

namespace sage {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

bool& pdl_chain_flag() {
  static thread_local bool flag = false;
  return flag;
}

}  // namespace sage

extern "C" unsigned long long sage_b200_launch_count(void) { return sage::g_launches.load(std::memory_order_relaxed); }

extern "C" int sage_b200_version(void) { return SAGE_B200_VERSION; }

extern "C" const char* sage_b200_last_error(void) { return sage::error_buffer(); }

// ---------------------------------------------------------------------------------------------
// The whole forward path in one call: K mean, Q/K quantisation, V cast, attention.  It only chains the
// entry points above over one caller-provided workspace, so a host pays one foreign call (and one
// allocation) per attention instead of five; at short sequences that host time is most of the step.
// ---------------------------------------------------------------------------------------------
namespace sage {
struct FwdPlan {
  size_t q8, k8, qs, ks, km, scratch, v16, total;     // byte offsets into the workspace, and its size
  int q_groups, k_groups;
  int q_warp, k_warp, q_kind, k_kind;
};
static size_t align_up(size_t x) { return (x + 255) & ~size_t(255); }

static FwdPlan fwd_plan(int dtype, int batch, int heads_q, int heads_kv, int len_q, int len_kv, int head_dim,
                        int blk_q, int blk_k, int warp_q, int warp_k, int granularity, int smooth_k, int cast_v) {
  FwdPlan p;
  const bool per_thread = (granularity == SAGE_B200_GRAN_PER_THREAD);
  p.q_kind = per_thread ? SAGE_B200_GROUP_Q_THREAD : SAGE_B200_GROUP_BLOCK;
  p.k_kind = per_thread ? SAGE_B200_GROUP_K_THREAD : SAGE_B200_GROUP_BLOCK;
  p.q_warp = per_thread ? warp_q : blk_q;
  p.k_warp = per_thread ? warp_k : blk_k;
  const int qb = (len_q + blk_q - 1) / blk_q, kb = (len_kv + blk_k - 1) / blk_k;
  p.q_groups = per_thread ? qb * (blk_q / warp_q) * 8 : qb;
  p.k_groups = per_thread ? kb * (blk_k / warp_k) * 4 : kb;
  size_t off = 0;
  p.q8 = off; off = align_up(off + size_t(batch) * heads_q * len_q * head_dim);
  p.k8 = off; off = align_up(off + size_t(batch) * heads_kv * len_kv * head_dim);
  p.qs = off; off = align_up(off + size_t(batch) * heads_q * p.q_groups * sizeof(float));
  p.ks = off; off = align_up(off + size_t(batch) * heads_kv * p.k_groups * sizeof(float));
  p.km = off; off = align_up(off + (smooth_k ? size_t(batch) * heads_kv * head_dim * 2 : 0));
  p.scratch = off; off = align_up(off + (smooth_k ? sage_b200_mean_k_scratch_bytes(batch, heads_kv, len_kv, head_dim) : 0));
  p.v16 = off; off = align_up(off + (cast_v ? size_t(batch) * heads_kv * len_kv * head_dim * 2 : 0));
  p.total = off;
  (void)dtype;
  return p;
}
}  // namespace sage

extern "C" size_t sage_b200_sageattn_workspace_bytes(int dtype, int batch, int heads_q, int heads_kv, int len_q,
                                                     int len_kv, int head_dim, int blk_q, int blk_k, int warp_q,
                                                     int warp_k, int granularity, int smooth_k, int cast_v) {
  if (batch <= 0 || heads_q <= 0 || heads_kv <= 0 || len_q <= 0 || len_kv <= 0 || head_dim <= 0 || blk_q <= 0 ||
      blk_k <= 0 || warp_q <= 0 || warp_k <= 0)
    return 0;
  return sage::fwd_plan(dtype, batch, heads_q, heads_kv, len_q, len_kv, head_dim, blk_q, blk_k, warp_q, warp_k,
                        granularity, smooth_k, cast_v).total;
}

extern "C" int sage_b200_sageattn(const void* q, const void* k, const void* v, void* out, float* lse, void* km_out,
                                  void* workspace, size_t workspace_bytes, int32_t* status, int dtype, int batch,
                                  int heads_q, int heads_kv, int len_q, int len_kv, int head_dim,
                                  const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                                  const int64_t o_strides[3], int is_causal, float sm_scale, int blk_q, int blk_k,
                                  int warp_q, int warp_k, int granularity, int smooth_k, int pv_accum, int div_mode,
                                  void* stream) {
  using namespace sage;
  SAGE_REQUIRE(q && k && v && out && workspace && q_strides && k_strides && v_strides && o_strides, "sageattn: null pointer");
  SAGE_REQUIRE(dtype == SAGE_B200_F16 || dtype == SAGE_B200_BF16, "sageattn: dtype must be fp16 or bf16");
  SAGE_REQUIRE(batch > 0 && heads_q > 0 && heads_kv > 0 && len_q > 0 && len_kv > 0, "sageattn: empty tensor");
  SAGE_REQUIRE(pv_accum == SAGE_B200_PV_F32 || pv_accum == SAGE_B200_PV_F16 || pv_accum == SAGE_B200_PV_F16_F32,
               "sageattn: pv_accum must be fp32, fp16 or fp16+fp32 (the fp8 and smoothed-V variants take their own calls)");
  SAGE_REQUIRE(granularity == SAGE_B200_GRAN_PER_THREAD || granularity == SAGE_B200_GRAN_PER_BLOCK,
               "sageattn: unknown granularity %d", granularity);
  SAGE_REQUIRE(blk_q > 0 && blk_k > 0 && warp_q > 0 && warp_k > 0, "sageattn: bad tile configuration");
  SAGE_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, "sageattn: workspace must be 256-byte aligned");
  // fp16 V with rows the tensor maps can address is read in place; anything else is cast into the workspace
  const bool v_in_place = dtype == SAGE_B200_F16 && (reinterpret_cast<uintptr_t>(v) & 15u) == 0 &&
                          v_strides[0] % 8 == 0 && v_strides[1] % 8 == 0 && v_strides[2] % 8 == 0;
  const FwdPlan p = fwd_plan(dtype, batch, heads_q, heads_kv, len_q, len_kv, head_dim, blk_q, blk_k, warp_q, warp_k,
                             granularity, smooth_k, v_in_place ? 0 : 1);
  SAGE_REQUIRE(workspace_bytes >= p.total, "sageattn: workspace too small (%zu < %zu bytes)", workspace_bytes, p.total);
  uint8_t* w = static_cast<uint8_t*>(workspace);
  int8_t* q8 = reinterpret_cast<int8_t*>(w + p.q8);
  int8_t* k8 = reinterpret_cast<int8_t*>(w + p.k8);
  float* qs = reinterpret_cast<float*>(w + p.qs);
  float* ks = reinterpret_cast<float*>(w + p.ks);
  void* km = smooth_k ? static_cast<void*>(w + p.km) : nullptr;
  // the quantised copies are (batch, heads, len, head_dim) contiguous
  const int64_t q8_st[3] = {int64_t(heads_q) * len_q * head_dim, int64_t(len_q) * head_dim, head_dim};
  const int64_t k8_st[3] = {int64_t(heads_kv) * len_kv * head_dim, int64_t(len_kv) * head_dim, head_dim};

  // the first kernel is an ordinary launch (it must not overtake whatever used this memory before);
  // every later one may be placed while its predecessor drains
  PdlChain chain;
  int rc = sage_b200_quant_int8(q, nullptr, q8, qs, dtype, batch, heads_q, len_q, head_dim, q_strides, q8_st, blk_q,
                                p.q_warp, p.q_kind, div_mode, stream);
  if (rc != SAGE_B200_OK) return rc;
  chain.arm();
  if (smooth_k) {
    rc = sage_b200_mean_k(k, km, w + p.scratch, p.v16 - p.scratch, dtype, batch, heads_kv, len_kv, head_dim, k_strides, stream);
    if (rc != SAGE_B200_OK) return rc;
    if (km_out != nullptr) {
      const cudaError_t e = cudaMemcpyAsync(km_out, km, size_t(batch) * heads_kv * head_dim * 2, cudaMemcpyDeviceToDevice,
                                            static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return fail(SAGE_B200_ERR_CUDA, "sageattn: copying the K mean failed: %s", cudaGetErrorString(e));
    }
  }
  rc = sage_b200_quant_int8(k, km, k8, ks, dtype, batch, heads_kv, len_kv, head_dim, k_strides, k8_st, blk_k, p.k_warp,
                            p.k_kind, div_mode, stream);
  if (rc != SAGE_B200_OK) return rc;
  const void* v16 = v;
  const int64_t* v16_st = v_strides;
  if (!v_in_place) {
    rc = sage_b200_cast_v_f16(v, w + p.v16, dtype, batch, heads_kv, len_kv, head_dim, v_strides, k8_st, stream);
    if (rc != SAGE_B200_OK) return rc;
    v16 = w + p.v16;
    v16_st = k8_st;                       // same shape and order as the quantised K
  }
  return sage_b200_attn_fwd(q8, k8, v16, out, qs, ks, lse, status, dtype, batch, heads_q, heads_kv, len_q, len_kv,
                            head_dim, q8_st, k8_st, v16_st, o_strides, is_causal, sm_scale, blk_q, blk_k, warp_q, warp_k,
                            granularity, pv_accum, stream);
}
