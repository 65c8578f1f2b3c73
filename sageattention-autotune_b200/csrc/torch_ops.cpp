// Torch operators of the B200 SageAttention path, registered from native code through torch's stable
// ABI (no libtorch symbols beyond the C shim, so one build serves every torch >= 2.10).
//
// The reference registers its kernels the same way: STABLE_TORCH_LIBRARY(sageattention_qattn_sm80, m)
// with one schema per accumulate mode (csrc/qattn/pybind_sm80.cpp:24-98, signatures
// csrc/qattn/attn_cuda_sm80.h:7-66) and takes the device guard and the current stream per call
// (csrc/utils.cuh:9-22).  The four attention operators below keep the reference's names and argument
// lists under the namespace `sageattention_b200`, so code written against
// torch.ops.sageattention_qattn_sm80.* runs on these kernels by swapping the namespace.  The rest of
// the namespace exposes the other C entry points of include/sage_b200.h (K mean, int8 quantisers, V
// cast / fp8 quantiser, the fp8 attention core and the whole forward call).
//
// Every operator is a thin shim: argument checks on the tensors, strides in (batch, head, sequence)
// order for either layout, the current CUDA stream of the tensor's device, then the C ABI of
// libsage_b200.so.  Fake (meta) implementations are registered from Python (sageattention/ops.py),
// as the reference does (sageattention/cuda_compile.py:9-68).
#include <cuda_runtime_api.h>
#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/csrc/stable/accelerator.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/ops.h>
#include <torch/csrc/stable/tensor.h>
#include <torch/headeronly/core/ScalarType.h>
#include <torch/headeronly/util/Exception.h>

#include <array>
#include <optional>
#include <tuple>
#include <vector>

#include "../../include/sage_b200.h"

namespace {

using torch::headeronly::ScalarType;
using torch::stable::Tensor;

struct Dims {
  int b, h, n, d;
};

// 0 = "NHD" (batch, seq, heads, dim), 1 = "HND" (batch, heads, seq, dim): the reference's encoding
// (csrc/qattn/qk_int8_sv_f16_launch_sm80.cuh:60-77)
Dims dims_of(const Tensor& t, int64_t layout) {
  STD_TORCH_CHECK(t.dim() == 4, "expected a 4-D tensor");
  STD_TORCH_CHECK(layout == 0 || layout == 1, "tensor_layout must be 0 (NHD) or 1 (HND)");
  if (layout == 1) return {int(t.size(0)), int(t.size(1)), int(t.size(2)), int(t.size(3))};
  return {int(t.size(0)), int(t.size(2)), int(t.size(1)), int(t.size(3))};
}
std::array<int64_t, 3> strides_of(const Tensor& t, int64_t layout) {
  if (layout == 1) return {t.stride(0), t.stride(1), t.stride(2)};
  return {t.stride(0), t.stride(2), t.stride(1)};
}
int dtype_code(const Tensor& t) {
  const ScalarType st = t.scalar_type();
  STD_TORCH_CHECK(st == ScalarType::Half || st == ScalarType::BFloat16, "expected an fp16 or bf16 tensor");
  return st == ScalarType::Half ? SAGE_B200_F16 : SAGE_B200_BF16;
}
void check_cuda_lastdim(const Tensor& t, const char* name) {
  STD_TORCH_CHECK(t.is_cuda(), "Tensor ", name, " must be on CUDA");
  STD_TORCH_CHECK(t.dim() == 4 && t.stride(3) == 1, "Tensor ", name, " must be 4-D with a contiguous last dimension");
}
void* stream_of(const Tensor& t) {
  void* s = nullptr;
  TORCH_ERROR_CODE_CHECK(aoti_torch_get_current_cuda_stream(t.get_device_index(), &s));
  return s;
}
void check_rc(int rc) { STD_TORCH_CHECK(rc == SAGE_B200_OK, "sage_b200 error ", rc, ": ", sage_b200_last_error()); }

std::vector<int64_t> shape_like(const Tensor& t) { return {t.size(0), t.size(1), t.size(2), t.size(3)}; }

// TMA and the 16-byte vector kernels need a 16-byte aligned base and strides that are multiples of
// 8 elements; anything else (a view that starts at an odd offset, odd strides) is copied once
Tensor aligned16(const Tensor& t) {
  const bool ok = (reinterpret_cast<uintptr_t>(t.const_data_ptr()) & 15u) == 0 && t.stride(0) % 8 == 0 &&
                  t.stride(1) % 8 == 0 && t.stride(2) % 8 == 0;
  return ok ? t : torch::stable::contiguous(t);
}

// ------------------------------------------------------------------------------------ attention core
Tensor attn_common(const Tensor& query, const Tensor& key, const Tensor& value, const Tensor& output,
                   const Tensor& query_scale, const Tensor& key_scale, const Tensor* value_mean,
                   const Tensor* value_scale, int64_t tensor_layout, bool is_causal, double sm_scale, int64_t blk_q,
                   int64_t blk_k, int64_t warp_q, int64_t warp_k, bool return_lse, int pv_accum, int64_t granularity) {
  check_cuda_lastdim(query, "query");
  check_cuda_lastdim(key, "key");
  check_cuda_lastdim(value, "value");
  check_cuda_lastdim(output, "output");
  STD_TORCH_CHECK(query.scalar_type() == ScalarType::Char && key.scalar_type() == ScalarType::Char,
                  "query and key must be int8");
  STD_TORCH_CHECK(query_scale.scalar_type() == ScalarType::Float && key_scale.scalar_type() == ScalarType::Float,
                  "query_scale and key_scale must be fp32");
  STD_TORCH_CHECK(query_scale.is_contiguous() && key_scale.is_contiguous(), "scales must be contiguous");
  const Dims q = dims_of(query, tensor_layout), k = dims_of(key, tensor_layout), v = dims_of(value, tensor_layout);
  const Dims o = dims_of(output, tensor_layout);
  STD_TORCH_CHECK(k.b == q.b && v.b == q.b && k.d == q.d && v.d == q.d && v.h == k.h && v.n == k.n,
                  "query, key and value shapes do not agree");
  STD_TORCH_CHECK(o.b == q.b && o.h == q.h && o.n == q.n && o.d == q.d, "output must have query's shape");
  const int out_dtype = dtype_code(output);
  const bool fp8 = value_scale != nullptr;
  STD_TORCH_CHECK(fp8 ? value.element_size() == 1 : value.scalar_type() == ScalarType::Half,
                  fp8 ? "value must be fp8 e4m3" : "value must be fp16");

  const torch::stable::accelerator::DeviceGuard guard(query.get_device_index());
  Tensor lse = return_lse ? torch::stable::new_empty(query, {int64_t(q.b), int64_t(q.h), int64_t(q.n)}, ScalarType::Float)
                          : torch::stable::new_empty(query, {0}, ScalarType::Float);
  const auto qs = strides_of(query, tensor_layout), ks = strides_of(key, tensor_layout);
  const auto vs = strides_of(value, tensor_layout), os = strides_of(output, tensor_layout);
  float* lse_ptr = return_lse ? static_cast<float*>(lse.data_ptr()) : nullptr;
  const auto* q8 = static_cast<const int8_t*>(query.const_data_ptr());
  const auto* k8 = static_cast<const int8_t*>(key.const_data_ptr());
  const auto* qsc = static_cast<const float*>(query_scale.const_data_ptr());
  const auto* ksc = static_cast<const float*>(key_scale.const_data_ptr());
  void* stream = stream_of(query);
  int rc;
  if (fp8) {
    STD_TORCH_CHECK(value_scale->scalar_type() == ScalarType::Float && value_scale->is_contiguous() &&
                        value_scale->numel() == int64_t(k.b) * k.h * k.d,
                    "value_scale must be contiguous fp32 (batch, kv_heads, head_dim)");
    rc = sage_b200_attn_fwd_fp8(q8, k8, value.const_data_ptr(), static_cast<const float*>(value_scale->const_data_ptr()),
                                output.data_ptr(), qsc, ksc, lse_ptr, nullptr, out_dtype, q.b, q.h, k.h, q.n, k.n, q.d,
                                qs.data(), ks.data(), vs.data(), os.data(), is_causal, float(sm_scale), int(blk_q),
                                int(blk_k), int(warp_q), int(warp_k), int(granularity), stream);
  } else if (value_mean != nullptr) {
    STD_TORCH_CHECK(value_mean->is_cuda() && value_mean->is_contiguous() && value_mean->dim() == 3 &&
                        value_mean->scalar_type() == output.scalar_type() &&
                        value_mean->numel() == int64_t(k.b) * k.h * k.d,
                    "value_mean must be contiguous (batch, kv_heads, head_dim) in the output dtype");
    rc = sage_b200_attn_fwd_fuse_v_mean(q8, k8, value.const_data_ptr(), value_mean->const_data_ptr(), output.data_ptr(),
                                        qsc, ksc, lse_ptr, nullptr, out_dtype, q.b, q.h, k.h, q.n, k.n, q.d, qs.data(),
                                        ks.data(), vs.data(), os.data(), is_causal, float(sm_scale), int(blk_q),
                                        int(blk_k), int(warp_q), int(warp_k), int(granularity), stream);
  } else {
    rc = sage_b200_attn_fwd(q8, k8, value.const_data_ptr(), output.data_ptr(), qsc, ksc, lse_ptr, nullptr, out_dtype,
                            q.b, q.h, k.h, q.n, k.n, q.d, qs.data(), ks.data(), vs.data(), os.data(), is_causal,
                            float(sm_scale), int(blk_q), int(blk_k), int(warp_q), int(warp_k), int(granularity),
                            pv_accum, stream);
  }
  check_rc(rc);
  return lse;
}

#define SAGE_ATTN_OP(name, mode)                                                                                   \
  Tensor name(const Tensor& query, const Tensor& key, const Tensor& value, const Tensor& output,                   \
              const Tensor& query_scale, const Tensor& key_scale, int64_t tensor_layout, bool is_causal,           \
              double sm_scale, int64_t blk_q, int64_t blk_k, int64_t warp_q, int64_t warp_k, bool return_lse) {    \
    return attn_common(query, key, value, output, query_scale, key_scale, nullptr, nullptr, tensor_layout,         \
                       is_causal, sm_scale, blk_q, blk_k, warp_q, warp_k, return_lse, mode,                        \
                       SAGE_B200_GRAN_PER_THREAD);                                                                 \
  }
SAGE_ATTN_OP(qk_int8_sv_f16_accum_f32_attn, SAGE_B200_PV_F32)
SAGE_ATTN_OP(qk_int8_sv_f16_accum_f16_attn, SAGE_B200_PV_F16)
SAGE_ATTN_OP(qk_int8_sv_f16_accum_f16_attn_inst_buf, SAGE_B200_PV_F16_F32)
#undef SAGE_ATTN_OP

Tensor qk_int8_sv_f16_accum_f16_fuse_v_mean_attn(const Tensor& query, const Tensor& key, const Tensor& value,
                                                 const Tensor& output, const Tensor& query_scale,
                                                 const Tensor& key_scale, const Tensor& value_mean,
                                                 int64_t tensor_layout, bool is_causal, double sm_scale,
                                                 int64_t blk_q, int64_t blk_k, int64_t warp_q, int64_t warp_k,
                                                 bool return_lse) {
  return attn_common(query, key, value, output, query_scale, key_scale, &value_mean, nullptr, tensor_layout, is_causal,
                     sm_scale, blk_q, blk_k, warp_q, warp_k, return_lse, SAGE_B200_PV_F16, SAGE_B200_GRAN_PER_THREAD);
}

// fp8 e4m3 P.V with one V scale per channel; no counterpart among the reference's registered operators
Tensor qk_int8_sv_f8_accum_f32_attn(const Tensor& query, const Tensor& key, const Tensor& value, const Tensor& output,
                                    const Tensor& query_scale, const Tensor& key_scale, const Tensor& value_scale,
                                    int64_t tensor_layout, bool is_causal, double sm_scale, int64_t blk_q,
                                    int64_t blk_k, int64_t warp_q, int64_t warp_k, bool return_lse) {
  return attn_common(query, key, value, output, query_scale, key_scale, nullptr, &value_scale, tensor_layout, is_causal,
                     sm_scale, blk_q, blk_k, warp_q, warp_k, return_lse, SAGE_B200_PV_F8, SAGE_B200_GRAN_PER_THREAD);
}

// the same three accumulate modes with one scale per BLKQ x D / BLKK x D tile (what the reference's
// Triton backend consumes); pv_accum: 0 fp32, 1 fp16, 2 fp16+fp32
Tensor qk_int8_sv_f16_attn_per_block(const Tensor& query, const Tensor& key, const Tensor& value,
                                     const Tensor& output, const Tensor& query_scale, const Tensor& key_scale,
                                     int64_t tensor_layout, bool is_causal, double sm_scale, int64_t blk_q,
                                     int64_t blk_k, int64_t pv_accum, bool return_lse) {
  STD_TORCH_CHECK(pv_accum >= 0 && pv_accum <= 2, "pv_accum must be 0 (fp32), 1 (fp16) or 2 (fp16+fp32)");
  return attn_common(query, key, value, output, query_scale, key_scale, nullptr, nullptr, tensor_layout, is_causal,
                     sm_scale, blk_q, blk_k, blk_q, blk_k, return_lse, int(pv_accum), SAGE_B200_GRAN_PER_BLOCK);
}

// ------------------------------------------------------------------------------------ front end
// k.mean(dim=seq, keepdim=True) in k's dtype (sageattention/cuda_attn.py:167-170)
Tensor mean_k(const Tensor& k_in, int64_t tensor_layout) {
  check_cuda_lastdim(k_in, "k");
  const Tensor k = aligned16(k_in);
  const Dims d = dims_of(k, tensor_layout);
  const int dt = dtype_code(k);
  const torch::stable::accelerator::DeviceGuard guard(k.get_device_index());
  const std::vector<int64_t> shape = tensor_layout == 1 ? std::vector<int64_t>{d.b, d.h, 1, d.d}
                                                         : std::vector<int64_t>{d.b, 1, d.h, d.d};
  Tensor km = torch::stable::new_empty(k, shape);
  const size_t nbytes = sage_b200_mean_k_scratch_bytes(d.b, d.h, d.n, d.d);
  Tensor scratch = torch::stable::new_empty(k, {int64_t(nbytes / 4 + 1)}, ScalarType::Float);
  const auto st = strides_of(k, tensor_layout);
  check_rc(sage_b200_mean_k(k.const_data_ptr(), km.data_ptr(), scratch.data_ptr(), nbytes, dt, d.b, d.h, d.n, d.d,
                            st.data(), stream_of(k)));
  return km;
}

// (int8 tensor, fp32 scales): group_kind 0 = Q per-thread, 1 = K per-thread, 2 = per block
// (sageattention/triton/quant_per_thread.py:118-205, quant_per_block.py:81-173)
std::tuple<Tensor, Tensor> quant_int8(const Tensor& x_in, const std::optional<Tensor>& mean, int64_t tensor_layout,
                                      int64_t blk, int64_t warp, int64_t group_kind, int64_t div_mode) {
  check_cuda_lastdim(x_in, "x");
  const Tensor x = aligned16(x_in);
  const Dims d = dims_of(x, tensor_layout);
  const int dt = dtype_code(x);
  STD_TORCH_CHECK(blk > 0 && warp > 0 && warp <= blk, "bad blk / warp");
  const int64_t blocks = (d.n + blk - 1) / blk;
  const int64_t groups = group_kind == SAGE_B200_GROUP_Q_THREAD   ? blocks * (blk / warp) * 8
                         : group_kind == SAGE_B200_GROUP_K_THREAD ? blocks * (blk / warp) * 4
                                                                  : blocks;
  const torch::stable::accelerator::DeviceGuard guard(x.get_device_index());
  Tensor out = torch::stable::new_empty(x, shape_like(x), ScalarType::Char);
  Tensor scale = torch::stable::new_empty(x, {int64_t(d.b), int64_t(d.h), groups}, ScalarType::Float);
  const void* mean_ptr = nullptr;
  Tensor mean_c = x;
  if (mean.has_value()) {
    STD_TORCH_CHECK(mean->scalar_type() == x.scalar_type() && mean->numel() == int64_t(d.b) * d.h * d.d,
                    "mean must have x's dtype and one value per (batch, head, channel)");
    mean_c = torch::stable::contiguous(*mean);
    mean_ptr = mean_c.const_data_ptr();
  }
  const auto xs = strides_of(x, tensor_layout), os = strides_of(out, tensor_layout);
  check_rc(sage_b200_quant_int8(x.const_data_ptr(), mean_ptr, static_cast<int8_t*>(out.data_ptr()),
                                static_cast<float*>(scale.data_ptr()), dt, d.b, d.h, d.n, d.d, xs.data(), os.data(),
                                int(blk), int(warp), int(group_kind), int(div_mode), stream_of(x)));
  return {out, scale};
}

// v.to(torch.float16) (sageattention/cuda_attn.py:195)
Tensor cast_v_f16(const Tensor& v_in, int64_t tensor_layout) {
  check_cuda_lastdim(v_in, "v");
  const Tensor v = aligned16(v_in);
  const Dims d = dims_of(v, tensor_layout);
  const int dt = dtype_code(v);
  const torch::stable::accelerator::DeviceGuard guard(v.get_device_index());
  Tensor out = torch::stable::new_empty(v, shape_like(v), ScalarType::Half);
  const auto vs = strides_of(v, tensor_layout), os = strides_of(out, tensor_layout);
  check_rc(sage_b200_cast_v_f16(v.const_data_ptr(), out.data_ptr(), dt, d.b, d.h, d.n, d.d, vs.data(), os.data(),
                                stream_of(v)));
  return out;
}

// (v as e4m3 bytes, fp32 scale per (batch, head, channel))
std::tuple<Tensor, Tensor> quant_v_fp8(const Tensor& v_in, int64_t tensor_layout) {
  check_cuda_lastdim(v_in, "v");
  const Tensor v = aligned16(v_in);
  const Dims d = dims_of(v, tensor_layout);
  const int dt = dtype_code(v);
  const torch::stable::accelerator::DeviceGuard guard(v.get_device_index());
  Tensor out = torch::stable::new_empty(v, shape_like(v), ScalarType::Float8_e4m3fn);
  Tensor scale = torch::stable::new_empty(v, {int64_t(d.b), int64_t(d.h), int64_t(d.d)}, ScalarType::Float);
  const size_t nbytes = sage_b200_quant_v_fp8_scratch_bytes(d.b, d.h, d.n, d.d);
  Tensor scratch = torch::stable::new_empty(v, {int64_t(nbytes / 4 + 1)}, ScalarType::Float);
  const auto vs = strides_of(v, tensor_layout), os = strides_of(out, tensor_layout);
  check_rc(sage_b200_quant_v_fp8(v.const_data_ptr(), out.data_ptr(), static_cast<float*>(scale.data_ptr()),
                                 scratch.data_ptr(), nbytes, dt, d.b, d.h, d.n, d.d, vs.data(), os.data(),
                                 stream_of(v)));
  return {out, scale};
}

// The whole forward path in one operator (sageattention/cuda_attn.py:126-274 from the K mean to the
// attention kernel).  Returns (output, lse, km): lse is base 2 without the smooth-k correction and
// empty unless return_lse; km is the K mean, empty unless smooth_k and return_lse.
std::tuple<Tensor, Tensor, Tensor> sageattn(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in,
                                            int64_t tensor_layout, bool is_causal, double sm_scale, int64_t blk_q,
                                            int64_t blk_k, int64_t warp_q, int64_t warp_k, int64_t granularity,
                                            bool smooth_k, int64_t pv_accum, int64_t div_mode, bool return_lse) {
  check_cuda_lastdim(q_in, "q");
  check_cuda_lastdim(k_in, "k");
  check_cuda_lastdim(v_in, "v");
  const Tensor q = aligned16(q_in), k = aligned16(k_in), v = aligned16(v_in);
  const Dims dq = dims_of(q, tensor_layout), dk = dims_of(k, tensor_layout), dv = dims_of(v, tensor_layout);
  const int dt = dtype_code(q);
  STD_TORCH_CHECK(dtype_code(k) == dt && dtype_code(v) == dt, "q, k and v must have the same dtype");
  STD_TORCH_CHECK(dk.b == dq.b && dk.d == dq.d && dv.b == dk.b && dv.h == dk.h && dv.n == dk.n && dv.d == dk.d,
                  "q, k and v shapes do not agree");
  const torch::stable::accelerator::DeviceGuard guard(q.get_device_index());
  const bool v_in_place = dt == SAGE_B200_F16 && (reinterpret_cast<uintptr_t>(v.const_data_ptr()) & 15u) == 0 &&
                          v.stride(0) % 8 == 0 && v.stride(1) % 8 == 0 && v.stride(2) % 8 == 0;
  const size_t nbytes = sage_b200_sageattn_workspace_bytes(dt, dq.b, dq.h, dk.h, dq.n, dk.n, dq.d, int(blk_q),
                                                           int(blk_k), int(warp_q), int(warp_k), int(granularity),
                                                           smooth_k, v_in_place ? 0 : 1);
  STD_TORCH_CHECK(nbytes > 0, "bad tile configuration");
  Tensor work = torch::stable::new_empty(q, {int64_t(nbytes)}, ScalarType::Byte);
  Tensor out = torch::stable::new_empty(q, shape_like(q));
  Tensor lse = return_lse ? torch::stable::new_empty(q, {int64_t(dq.b), int64_t(dq.h), int64_t(dq.n)}, ScalarType::Float)
                          : torch::stable::new_empty(q, {0}, ScalarType::Float);
  const bool want_km = smooth_k && return_lse;
  const std::vector<int64_t> km_shape = !want_km              ? std::vector<int64_t>{0}
                                        : tensor_layout == 1 ? std::vector<int64_t>{dk.b, dk.h, 1, dk.d}
                                                             : std::vector<int64_t>{dk.b, 1, dk.h, dk.d};
  Tensor km = torch::stable::new_empty(k, km_shape);
  const auto qs = strides_of(q, tensor_layout), ks = strides_of(k, tensor_layout), vs = strides_of(v, tensor_layout);
  const auto os = strides_of(out, tensor_layout);
  check_rc(sage_b200_sageattn(q.const_data_ptr(), k.const_data_ptr(), v.const_data_ptr(), out.data_ptr(),
                              return_lse ? static_cast<float*>(lse.data_ptr()) : nullptr,
                              want_km ? km.data_ptr() : nullptr, work.data_ptr(), nbytes, nullptr, dt, dq.b, dq.h, dk.h,
                              dq.n, dk.n, dq.d, qs.data(), ks.data(), vs.data(), os.data(), is_causal, float(sm_scale),
                              int(blk_q), int(blk_k), int(warp_q), int(warp_k), int(granularity), smooth_k,
                              int(pv_accum), int(div_mode), stream_of(q)));
  return {out, lse, km};
}

}  // namespace

#define SAGE_ATTN_SCHEMA(name, extra)                                                                          \
  #name "(Tensor query, Tensor key, Tensor value, Tensor(a!) output, Tensor query_scale, Tensor key_scale, "   \
        extra "int tensor_layout, bool is_causal, float sm_scale, int blk_q, int blk_k, int warp_q, int warp_k, " \
        "bool return_lse) -> Tensor"

STABLE_TORCH_LIBRARY(sageattention_b200, m) {
  m.def(SAGE_ATTN_SCHEMA(qk_int8_sv_f16_accum_f32_attn, ""));
  m.def(SAGE_ATTN_SCHEMA(qk_int8_sv_f16_accum_f16_attn, ""));
  m.def(SAGE_ATTN_SCHEMA(qk_int8_sv_f16_accum_f16_attn_inst_buf, ""));
  m.def(SAGE_ATTN_SCHEMA(qk_int8_sv_f16_accum_f16_fuse_v_mean_attn, "Tensor value_mean, "));
  m.def(SAGE_ATTN_SCHEMA(qk_int8_sv_f8_accum_f32_attn, "Tensor value_scale, "));
  m.def("qk_int8_sv_f16_attn_per_block(Tensor query, Tensor key, Tensor value, Tensor(a!) output, Tensor query_scale, "
        "Tensor key_scale, int tensor_layout, bool is_causal, float sm_scale, int blk_q, int blk_k, int pv_accum, "
        "bool return_lse) -> Tensor");
  m.def("mean_k(Tensor k, int tensor_layout) -> Tensor");
  m.def("quant_int8(Tensor x, Tensor? mean, int tensor_layout, int blk, int warp, int group_kind, int div_mode) "
        "-> (Tensor, Tensor)");
  m.def("cast_v_f16(Tensor v, int tensor_layout) -> Tensor");
  m.def("quant_v_fp8(Tensor v, int tensor_layout) -> (Tensor, Tensor)");
  m.def("sageattn(Tensor q, Tensor k, Tensor v, int tensor_layout, bool is_causal, float sm_scale, int blk_q, "
        "int blk_k, int warp_q, int warp_k, int granularity, bool smooth_k, int pv_accum, int div_mode, "
        "bool return_lse) -> (Tensor, Tensor, Tensor)");
}

STABLE_TORCH_LIBRARY_IMPL(sageattention_b200, CUDA, m) {
  m.impl("qk_int8_sv_f16_accum_f32_attn", TORCH_BOX(qk_int8_sv_f16_accum_f32_attn));
  m.impl("qk_int8_sv_f16_accum_f16_attn", TORCH_BOX(qk_int8_sv_f16_accum_f16_attn));
  m.impl("qk_int8_sv_f16_accum_f16_attn_inst_buf", TORCH_BOX(qk_int8_sv_f16_accum_f16_attn_inst_buf));
  m.impl("qk_int8_sv_f16_accum_f16_fuse_v_mean_attn", TORCH_BOX(qk_int8_sv_f16_accum_f16_fuse_v_mean_attn));
  m.impl("qk_int8_sv_f8_accum_f32_attn", TORCH_BOX(qk_int8_sv_f8_accum_f32_attn));
  m.impl("qk_int8_sv_f16_attn_per_block", TORCH_BOX(qk_int8_sv_f16_attn_per_block));
  m.impl("mean_k", TORCH_BOX(mean_k));
  m.impl("quant_int8", TORCH_BOX(quant_int8));
  m.impl("cast_v_f16", TORCH_BOX(cast_v_f16));
  m.impl("quant_v_fp8", TORCH_BOX(quant_v_fp8));
  m.impl("sageattn", TORCH_BOX(sageattn));
}
