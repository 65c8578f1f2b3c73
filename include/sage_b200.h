/*
 * sage_b200.h - C ABI of the B200 (sm_100a) SageAttention forward path.
 *
 * Every entry point takes plain device pointers, sizes, element strides and a
 * CUDA stream (passed as void*, i.e. a cudaStream_t); nothing here depends on
 * torch.  All functions return SAGE_B200_OK (0) or a negative error code and leave a
 * human-readable message retrievable with sage_b200_last_error() (thread-local).
 * Nothing is allocated or freed on the caller's behalf; kernels are enqueued on the
 * given stream and the call returns without synchronising.
 *
 * Tensor convention: a "4-D tensor" is addressed as
 *     base + b*stride[0] + h*stride[1] + n*stride[2] + d          (d contiguous)
 * with strides in ELEMENTS, which covers both layouts of the reference
 * ("NHD" = (B,N,H,D) and "HND" = (B,H,N,D), sageattention/cuda_attn.py:156-165).
 *
 * Each declaration cites the interface of the reference
 * (woct0rdho/sageattention-autotune) that it replaces.
 */
#ifndef SAGE_B200_H_
#define SAGE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAGE_B200_VERSION 100

/* error codes */
#define SAGE_B200_OK               0
#define SAGE_B200_ERR_INVALID     -1   /* bad argument (shape, dtype, stride, alignment) */
#define SAGE_B200_ERR_UNSUPPORTED -2   /* valid in the reference, not built here yet */
#define SAGE_B200_ERR_CUDA        -3   /* a CUDA runtime/driver call failed */
#define SAGE_B200_ERR_DEVICE      -4   /* the kernel reported a device-side failure (bounded wait ran out) */

/* element types of the 16-bit tensors */
#define SAGE_B200_F16  0
#define SAGE_B200_BF16 1

/* which rows share one int8 scale (sage_b200_quant_int8: group_kind) */
#define SAGE_B200_GROUP_Q_THREAD 0  /* reference Q grouping: rows r with equal r%8 inside a WARPQ-row block */
#define SAGE_B200_GROUP_K_THREAD 1  /* reference K grouping: row pairs, (r%8)/2, inside a WARPK-row block */
#define SAGE_B200_GROUP_BLOCK    2  /* one scale per BLK x D tile */

/* how x/scale is evaluated */
#define SAGE_B200_DIV_FULL 0   /* div.full.f32, what the reference's Triton kernels compile to on a GPU */
#define SAGE_B200_DIV_IEEE 1   /* correctly rounded, what a CPU evaluation of the same source gives */

/* scale granularity the attention kernel assumes (must match how Q/K were quantised) */
#define SAGE_B200_GRAN_PER_THREAD 0
#define SAGE_B200_GRAN_PER_BLOCK  1

/* accumulation mode of P.V (pv_accum_dtype of the reference API) */
#define SAGE_B200_PV_F32     0   /* "fp32"      */
#define SAGE_B200_PV_F16     1   /* "fp16"      */
#define SAGE_B200_PV_F16_F32 2   /* "fp16+fp32" */
#define SAGE_B200_PV_F8      3   /* fp8 e4m3 P and V, fp32 accumulate (sage_b200_attn_fwd_fp8 only) */

/* kernels of the attention core (sage_b200_tile_entry.kernel) */
#define SAGE_B200_KERNEL_TWO_TILE         0  /* 256 query rows per CTA share every K/V block; O accumulates in tensor memory */
#define SAGE_B200_KERNEL_ONE_TILE_FOLD    1  /* 128 query rows per CTA, fp16 partial products folded into fp32 by a fold warpgroup */
#define SAGE_B200_KERNEL_TWO_TILE_COUPLED 2  /* the two-level mode inside the two-tile kernel's softmax warps */
#define SAGE_B200_KERNEL_ONE_TILE_PERSISTENT 3  /* the one-tile kernel as one CTA per SM walking over the query tiles */

/*
 * One entry of the fixed tile table.  Replaces the reference's run-time selection among
 * _AUTOTUNE_CONFIGS (sageattention/cuda_autotune.py:9-41): the scale grouping a problem is quantised
 * and attended with, and the kernel configuration that runs it, chosen from measurements on B200.
 */
typedef struct sage_b200_tile_entry {
  int blk_q, blk_k, warp_q, warp_k;  /* which query rows and keys share an int8 scale */
  int kernel;                        /* SAGE_B200_KERNEL_* */
  int q_tiles_per_cta;               /* 128-row query tiles per CTA */
  int seq_bucket;                    /* index of the key-length bucket the entry was looked up in */
} sage_b200_tile_entry;

/* head_dim 64 / 128 / 256 (after padding), pv_accum one of SAGE_B200_PV_*.  Returns SAGE_B200_OK or
 * SAGE_B200_ERR_INVALID.  sage_b200_attn_fwd consults the same table for the kernel and the tiles per
 * CTA; the grouping is the caller's to pass to the quantisers and to sage_b200_attn_fwd alike. */
int sage_b200_tile_lookup(int head_dim, int is_causal, int pv_accum, int len_kv, sage_b200_tile_entry* entry);

int sage_b200_version(void);
const char* sage_b200_last_error(void);
/* Number of kernels this library has launched in this process so far (all threads, all devices).  The
 * reference has no counterpart; benchmarks use it to state how many of the library's own kernels ran
 * inside a timed region. */
unsigned long long sage_b200_launch_count(void);

/*
 * Channel mean of K over the sequence, rounded to K's dtype.
 * Replaces `km = k.mean(dim=seq_dim, keepdim=True)` (sageattention/cuda_attn.py:167-170).
 *   k        16-bit (batch, heads, len, head_dim) by strides
 *   km       out, (batch, heads, head_dim) contiguous, same dtype as k
 *   scratch  device buffer of at least sage_b200_mean_k_scratch_bytes(...) bytes holding
 *            the per-slice fp32 partial sums of the two-stage reduction
 */
size_t sage_b200_mean_k_scratch_bytes(int batch, int heads, int len, int head_dim);
int sage_b200_mean_k(const void* k, void* km, void* scratch, size_t scratch_bytes, int dtype,
                     int batch, int heads, int len, int head_dim, const int64_t k_strides[3],
                     void* stream);

/*
 * Channel mean of K for callers that must not allocate.  (No counterpart in the reference: it was
 * added for hosts that cannot call cudaMalloc around this library - code running inside a CUDA
 * graph capture or a stream-ordered region where allocation is forbidden, plugins handed a fixed
 * memory budget, and real-time loops that may not touch the allocator.)
 * Same result as sage_b200_mean_k, bit for bit; the partial sums of the two-stage reduction live in
 * a buffer built into the library (sage_b200_mean_k_static_capacity_bytes() = 2 MiB, held by every GPU
 * that loads the library until the process exits).  A shape whose partial sums do not fit is refused
 * with SAGE_B200_ERR_INVALID; sage_b200_mean_k_scratch_bytes(...) tells how much a shape needs.
 * The first call on each device looks up the buffer's device address (cudaGetSymbolAddress); make
 * that first call outside any stream capture.  No cudaMalloc/cudaFree or allocating library routine
 * is called.  All calls on a device share the one buffer: the kernels overwrite all of it that they
 * read, nothing needs clearing, but two calls that overlap on the GPU (different streams) race.
 */
size_t sage_b200_mean_k_static_capacity_bytes(void);
int sage_b200_mean_k_static(const void* k, void* km, int dtype, int batch, int heads, int len,
                            int head_dim, const int64_t k_strides[3], void* stream);

/*
 * int8 quantisation of Q or K with fp32 scales.
 * Replaces quant_query_per_thread_int8_kernel / quant_key_per_thread_int8_kernel
 * (sageattention/triton/quant_per_thread.py:22-115, host wrapper :118-205) and
 * quant_per_block_int8_kernel (sageattention/triton/quant_per_block.py:32-78, :81-173).
 *   x        16-bit input by strides;  mean: (batch, heads, head_dim) contiguous or NULL
 *   out      int8, same logical shape, by out_strides
 *   scale    fp32 (batch, heads, groups) contiguous with
 *            groups = ceil(len/blk) * (blk/warp) * {8 | 4}   for the two per-thread kinds,
 *            groups = ceil(len/blk)                           for SAGE_B200_GROUP_BLOCK
 *   blk      BLKQ or BLKK of the attention tile config (16, 32, 64 or 128; 16 serves per-warp Q scales with WARPQ = 16)
 *   warp     WARPQ or WARPK (8..blk, a power of two); ignored for SAGE_B200_GROUP_BLOCK
 * Rows past `len` inside the last block behave like the reference's masked loads:
 * they read as 0, the mean is still subtracted from them, they enter the maximum and
 * are not stored.
 */
int sage_b200_quant_int8(const void* x, const void* mean, int8_t* out, float* scale, int dtype,
                         int batch, int heads, int len, int head_dim,
                         const int64_t x_strides[3], const int64_t out_strides[3],
                         int blk, int warp, int group_kind, int div_mode, void* stream);

/*
 * K smoothing and quantisation in one call: channel mean of K (as sage_b200_mean_k) followed by the
 * int8 quantisation of K - mean (as sage_b200_quant_int8 with the K per-thread or per-block
 * grouping).  Replaces `km = k.mean(...)` plus the K half of per_thread_int8 / per_block_int8
 * (sageattention/cuda_attn.py:167-187, sageattention/triton/quant_per_thread.py:182-203).
 * `slice_bytes` = 0 runs the two steps over the whole tensor.  A non-zero value processes K in slices
 * of whole batches (or of heads when batch == 1) of about that many bytes, mean then quantise per
 * slice, so that the second read of a slice can hit the L2 cache.  On B200 this does not pay: at
 * 64 x 32768 x 128 fp16 the call takes 0.32 ms unsliced, 0.38 ms in 128 MiB slices and 0.46 ms in
 * 64 MiB slices, because every slice costs three more launches than it saves in HBM time.  Results do
 * not depend on the slicing, and km equals what sage_b200_mean_k gives for the whole tensor.
 *   km      out, (batch, heads, head_dim) contiguous, K's dtype
 *   scratch at least sage_b200_smooth_quant_k_scratch_bytes(...) bytes
 */
size_t sage_b200_smooth_quant_k_scratch_bytes(int batch, int heads, int len, int head_dim, size_t slice_bytes);
int sage_b200_smooth_quant_k(const void* k, void* km, int8_t* out, float* scale, void* scratch,
                             size_t scratch_bytes, int dtype, int batch, int heads, int len, int head_dim,
                             const int64_t k_strides[3], const int64_t out_strides[3], int blk, int warp,
                             int group_kind, int div_mode, size_t slice_bytes, void* stream);

/*
 * V cast to fp16.  Replaces `v.to(torch.float16)` (sageattention/cuda_attn.py:195,233,250).
 */
int sage_b200_cast_v_f16(const void* v, void* out, int dtype, int batch, int heads, int len,
                         int head_dim, const int64_t v_strides[3], const int64_t out_strides[3],
                         void* stream);

/*
 * V smoothing for the fp16 accumulator: out = fp16(v - v_mean), the difference rounded to V's dtype
 * first, as `(v - vm.unsqueeze(seq)).to(torch.float16)` does (sageattention/cuda_attn.py:209-211).
 * `v_mean` is the channel mean over the sequence, (batch, heads, head_dim) contiguous in V's dtype:
 * `v.mean(dim=seq)`, which sage_b200_mean_k computes for any (batch, heads, len, head_dim) tensor.
 */
int sage_b200_smooth_v_f16(const void* v, const void* v_mean, void* out, int dtype, int batch, int heads,
                           int len, int head_dim, const int64_t v_strides[3], const int64_t out_strides[3],
                           void* stream);

/*
 * Attention core on quantised Q/K and fp16 V.
 * Replaces torch.ops.sageattention_qattn_sm80.qk_int8_sv_f16_accum_f32_attn,
 * ..._accum_f16_attn and ..._accum_f16_attn_inst_buf (csrc/qattn/pybind_sm80.cpp:24-98,
 * csrc/qattn/qk_int8_sv_f16_launch_sm80.cuh:244-308), selected by `pv_accum`.
 *   q, k       int8 by strides;  v: fp16 by strides;  out: out_dtype by strides
 *   q_scale    fp32 (batch, heads_q, q_groups), k_scale fp32 (batch, heads_kv, k_groups), laid
 *              out as sage_b200_quant_int8 writes them for (blk_q, warp_q) / (blk_k, warp_k)
 *   lse        NULL, or fp32 (batch, heads_q, len_q): log2(sum) + max in base 2, as the
 *              reference kernel defines it (qk_int8_sv_f16_kernel_sm80.cuh:645-656)
 *   status     NULL, or 4 int32 the GPU can write (device memory, or pinned host memory, which a
 *              host can poll without synchronising), zeroed by the caller; if one of the kernel's
 *              bounded waits runs out, the first CTA to give up writes {code, blockIdx.x, .y, .z}
 *              there (code 10-69 = the wait that ran out, 99 = a CTA that started after another one
 *              had given up).  With or without a status word a CTA that gives up fills its rows of
 *              `out` with NaN, and the remaining CTAs of that launch return at once
 *   causal     top-left aligned: key j is visible to query i iff j <= i
 *   head_dim   64, 128 or 256 (the reference's dispatch, csrc/dispatch_utils.h:34-47)
 *   blk_k, warp_k  64 or 32, warp_k = blk_k
 * The same inputs give the same bits on every call.
 */
int sage_b200_attn_fwd(const int8_t* q, const int8_t* k, const void* v, void* out,
                       const float* q_scale, const float* k_scale, float* lse, int32_t* status,
                       int out_dtype, int batch, int heads_q, int heads_kv, int len_q, int len_kv,
                       int head_dim, const int64_t q_strides[3], const int64_t k_strides[3],
                       const int64_t v_strides[3], const int64_t o_strides[3], int is_causal,
                       float sm_scale, int blk_q, int blk_k, int warp_q, int warp_k,
                       int granularity, int pv_accum, void* stream);

/*
 * Budget of every bounded wait inside the attention kernels, in SM clocks, for launches made after
 * the call (process-wide; the default, about two seconds, is restored by a value <= 0).  Returns the
 * previous budget.  The reference has nothing comparable (its launcher does not even check the
 * launch, csrc/qattn/qk_int8_sv_f16_launch_sm80.cuh:193-209); hosts with a watchdog shorter than two
 * seconds lower it, and tests use a tiny value to drive the give-up path without faulting the GPU.
 */
long long sage_b200_set_wait_budget(long long cycles);

/*
 * The same with fp16 accumulation of a smoothed V and the channel mean added back to the normalised
 * output, in the output type.  Replaces `qk_int8_sv_f16_accum_f16_fuse_v_mean_attn`
 * (csrc/qattn/pybind_sm80.cpp:73-89, kernel csrc/qattn/qk_int8_sv_f16_kernel_sm80.cuh:551-569).
 *   v       the smoothed V (sage_b200_smooth_v_f16), fp16
 *   v_mean  (batch, heads_kv, head_dim) contiguous, in the OUTPUT dtype, 16-byte aligned
 */
int sage_b200_attn_fwd_fuse_v_mean(const int8_t* q, const int8_t* k, const void* v, const void* v_mean,
                                   void* out, const float* q_scale, const float* k_scale, float* lse,
                                   int32_t* status, int out_dtype, int batch, int heads_q, int heads_kv,
                                   int len_q, int len_kv, int head_dim, const int64_t q_strides[3],
                                   const int64_t k_strides[3], const int64_t v_strides[3],
                                   const int64_t o_strides[3], int is_causal, float sm_scale, int blk_q,
                                   int blk_k, int warp_q, int warp_k, int granularity, void* stream);

/*
 * The whole forward path in one call: `sageattn_qk_int8_pv_fp16_cuda` / `_sageattn_configured`
 * (sageattention/cuda_attn.py:126-274) from the K mean to the attention kernel, i.e.
 * sage_b200_quant_int8 (Q), sage_b200_mean_k + sage_b200_quant_int8 (K), sage_b200_cast_v_f16 when V is
 * not fp16 (or not addressable in place) and sage_b200_attn_fwd, chained on `stream` over one
 * caller-provided workspace of sage_b200_sageattn_workspace_bytes(...) bytes, 256-byte aligned
 * (pass cast_v = 1 there unless V is fp16 with 16-byte aligned rows).  One foreign call per attention
 * instead of five: at short sequences the host time of the separate calls is most of the step.
 *   q, k, v, out  16-bit tensors by strides, already padded to head_dim 64 / 128 / 256; out has q's dtype
 *   lse           NULL or fp32 (batch, heads_q, len_q), base 2, WITHOUT the smooth-k correction
 *   km_out        NULL, or (batch, heads_kv, head_dim) in K's dtype: receives the K mean (callers that
 *                 return the LSE need it for the correction q.km^T, sageattention/utils.py:39-49)
 *   pv_accum      SAGE_B200_PV_F32, _F16 or _F16_F32
 */
size_t sage_b200_sageattn_workspace_bytes(int dtype, int batch, int heads_q, int heads_kv, int len_q, int len_kv,
                                          int head_dim, int blk_q, int blk_k, int warp_q, int warp_k,
                                          int granularity, int smooth_k, int cast_v);
int sage_b200_sageattn(const void* q, const void* k, const void* v, void* out, float* lse, void* km_out,
                       void* workspace, size_t workspace_bytes, int32_t* status, int dtype, int batch,
                       int heads_q, int heads_kv, int len_q, int len_kv, int head_dim,
                       const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                       const int64_t o_strides[3], int is_causal, float sm_scale, int blk_q, int blk_k,
                       int warp_q, int warp_k, int granularity, int smooth_k, int pv_accum, int div_mode,
                       void* stream);

/*
 * V in fp8 e4m3 with one fp32 scale per (batch, head, channel): scale = max|v| over the sequence / 448,
 * v_fp8 = e4m3(v / scale), round to nearest, saturating.  The reference has no fp8 path in this
 * tree (sageattention/core.py:18-21 exports sageattn_qk_int8_pv_fp8_cuda = None; the kernels live on
 * an un-vendored branch), so this follows the published SageAttention2 scheme (per-channel V scale).
 *   v        16-bit input by strides;  out: 1 byte per element by out_strides (head_dim contiguous)
 *   v_scale  out, fp32 (batch, heads, head_dim) contiguous
 *   scratch  at least sage_b200_quant_v_fp8_scratch_bytes(...) bytes (per-slice channel maxima)
 */
size_t sage_b200_quant_v_fp8_scratch_bytes(int batch, int heads, int len, int head_dim);
int sage_b200_quant_v_fp8(const void* v, void* out, float* v_scale, void* scratch, size_t scratch_bytes,
                          int dtype, int batch, int heads, int len, int head_dim, const int64_t v_strides[3],
                          const int64_t out_strides[3], void* stream);

/*
 * Attention core with fp8 P.V: same as sage_b200_attn_fwd with pv_accum = SAGE_B200_PV_F8, plus
 *   v        fp8 e4m3 by strides (as written by sage_b200_quant_v_fp8)
 *   v_scale  fp32 (batch, heads_kv, head_dim) contiguous
 * P is scaled by 448 before it is rounded to e4m3 (the factor cancels between O and the row sum),
 * the accumulator is fp32.  No counterpart in this reference tree (see sage_b200_quant_v_fp8).
 */
int sage_b200_attn_fwd_fp8(const int8_t* q, const int8_t* k, const void* v, const float* v_scale, void* out,
                           const float* q_scale, const float* k_scale, float* lse, int32_t* status,
                           int out_dtype, int batch, int heads_q, int heads_kv, int len_q, int len_kv,
                           int head_dim, const int64_t q_strides[3], const int64_t k_strides[3],
                           const int64_t v_strides[3], const int64_t o_strides[3], int is_causal,
                           float sm_scale, int blk_q, int blk_k, int warp_q, int warp_k, int granularity,
                           void* stream);

/*
 * Head sharding over the GPUs of one node, one process per GPU, with the exchange of the output fused
 * into the attention epilogue.  The reference is single-GPU (its launcher writes one output tensor,
 * csrc/qattn/qk_int8_sv_f16_launch_sm80.cuh:138-209); these entry points have no counterpart there.
 *
 * Every process allocates one buffer for the WHOLE output with sage_b200_peer_alloc, sends the 64-byte
 * handle to the other processes (any host channel) and maps theirs with sage_b200_peer_open.  A thread
 * then names the other ranks' buffers with sage_b200_set_output_peers: byte_offsets[i] = (peer i's
 * mapped base) - (own base).  From then on every attention launch of that thread whose `out` lies in
 * the own buffer stores each finished row to out + byte_offsets[i] as well, with plain 32-byte stores
 * over NVLink, until the set is cleared with n = 0.  The stores of a launch have been performed when
 * the launch has completed; the ranks still have to meet (a barrier or any collective on the same
 * streams) before one reads what another wrote.  With peers set, `out` must be 32-byte aligned and its
 * strides multiples of 16 elements.  n <= 7.  Rows a CTA gives up on read as NaN in every copy.
 */
#define SAGE_B200_PEER_HANDLE_BYTES 64
int sage_b200_peer_alloc(size_t bytes, void** ptr, unsigned char* handle /* [64] out */);
int sage_b200_peer_open(const unsigned char* handle /* [64] */, void** ptr);
int sage_b200_peer_close(void* ptr);   /* a pointer from sage_b200_peer_open */
int sage_b200_peer_free(void* ptr);    /* a pointer from sage_b200_peer_alloc, after every peer closed it */
int sage_b200_set_output_peers(int n, const int64_t* byte_offsets);

#ifdef __cplusplus
}
#endif
#endif /* SAGE_B200_H_ */
