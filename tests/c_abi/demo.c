/* A C caller of the C ABI, with no Python and no torch in the process: fills Q, K, V on the host,
 * runs the whole forward path through sage_b200_sageattn on the current device, and checks the result
 * against a plain fp32 attention computed here.  Built and run by tests/test_c_abi_gpu.py:
 *     nvcc -x c demo.c -I<repo>/include -L<libdir> -lsage_b200 -lcudart -lm -o demo && ./demo
 * Exit code 0 = pass.  (TEST INFRASTRUCTURE.) */
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "sage_b200.h"

#define CHECK_CUDA(x)                                                                  \
  do {                                                                                 \
    cudaError_t e_ = (x);                                                              \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
      return 2;                                                                        \
    }                                                                                  \
  } while (0)

/* IEEE half <-> float, round to nearest even, enough for test data in [-8, 8] */
static uint16_t f2h(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (exp <= 0) return (uint16_t)sign; /* flush tiny values: not used by the test data */
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  uint32_t h = sign | ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
  return (uint16_t)h;
}
static float h2f(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
  uint32_t x;
  if (exp == 0) {
    if (man == 0) { x = sign; }
    else { float f = (float)man * (1.0f / 16777216.0f); memcpy(&x, &f, 4); x |= sign; }
  } else if (exp == 31) x = sign | 0x7f800000u | (man << 13);
  else x = sign | ((exp - 15 + 127) << 23) | (man << 13);
  float f;
  memcpy(&f, &x, 4);
  return f;
}
static uint32_t lcg(uint32_t* s) { *s = *s * 1664525u + 1013904223u; return *s; }
/* roughly normal: sum of four uniforms */
static float rnd(uint32_t* s) {
  float a = 0.0f;
  for (int i = 0; i < 4; ++i) a += (float)(lcg(s) >> 8) * (1.0f / 16777216.0f);
  return (a - 2.0f) * 1.7320508f;
}

int main(void) {
  const int B = 1, Hq = 4, Hkv = 2, N = 384, D = 64, causal = 1;
  const int blk_q = 128, blk_k = 64, warp_q = 32, warp_k = 64;
  const size_t nq = (size_t)B * Hq * N * D, nk = (size_t)B * Hkv * N * D;
  uint16_t* hq = malloc(nq * 2); uint16_t* hk = malloc(nk * 2); uint16_t* hv = malloc(nk * 2); uint16_t* ho = malloc(nq * 2);
  uint16_t* ho2 = malloc(nq * 2);
  float* ref = malloc(nq * 4);
  if (!hq || !hk || !hv || !ho || !ho2 || !ref) return 2;
  uint32_t seed = 12345u;
  for (size_t i = 0; i < nq; ++i) hq[i] = f2h(rnd(&seed));
  for (size_t i = 0; i < nk; ++i) hk[i] = f2h(rnd(&seed) + 1.5f * (float)((int)((i % D) % 3) - 1));   /* a channel offset for smooth_k */
  for (size_t i = 0; i < nk; ++i) hv[i] = f2h(rnd(&seed));

  /* fp32 reference, (batch, heads, len, dim) layout, GQA: q-head h uses kv-head h / (Hq/Hkv) */
  const float sm_scale = 1.0f / sqrtf((float)D);
  float* p = malloc((size_t)N * 4);
  for (int h = 0; h < Hq; ++h) {
    const int hk_i = h / (Hq / Hkv);
    for (int i = 0; i < N; ++i) {
      const int lim = causal ? i : N - 1;
      float m = -1e30f;
      for (int j = 0; j <= lim; ++j) {
        float s = 0.0f;
        for (int d = 0; d < D; ++d) s += h2f(hq[((size_t)h * N + i) * D + d]) * h2f(hk[((size_t)hk_i * N + j) * D + d]);
        p[j] = s * sm_scale;
        if (p[j] > m) m = p[j];
      }
      float sum = 0.0f;
      for (int j = 0; j <= lim; ++j) { p[j] = expf(p[j] - m); sum += p[j]; }
      for (int d = 0; d < D; ++d) {
        float acc = 0.0f;
        for (int j = 0; j <= lim; ++j) acc += p[j] * h2f(hv[((size_t)hk_i * N + j) * D + d]);
        ref[((size_t)h * N + i) * D + d] = acc / sum;
      }
    }
  }

  void *dq, *dk, *dv, *dout, *work;
  int32_t* dstatus;
  CHECK_CUDA(cudaMalloc(&dq, nq * 2)); CHECK_CUDA(cudaMalloc(&dk, nk * 2)); CHECK_CUDA(cudaMalloc(&dv, nk * 2));
  CHECK_CUDA(cudaMalloc(&dout, nq * 2)); CHECK_CUDA(cudaMalloc((void**)&dstatus, 16));
  CHECK_CUDA(cudaMemcpy(dq, hq, nq * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dk, hk, nk * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dv, hv, nk * 2, cudaMemcpyHostToDevice));
  const size_t wbytes = sage_b200_sageattn_workspace_bytes(SAGE_B200_F16, B, Hq, Hkv, N, N, D, blk_q, blk_k, warp_q, warp_k,
                                                           SAGE_B200_GRAN_PER_THREAD, 1, 0);
  if (wbytes == 0) { fprintf(stderr, "workspace size is 0\n"); return 1; }
  CHECK_CUDA(cudaMalloc(&work, wbytes));
  const int64_t sq[3] = {(int64_t)Hq * N * D, (int64_t)N * D, D}, sk[3] = {(int64_t)Hkv * N * D, (int64_t)N * D, D};
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));
  const int modes[3] = {SAGE_B200_PV_F32, SAGE_B200_PV_F16_F32, SAGE_B200_PV_F16};
  int failures = 0;
  for (int mi = 0; mi < 3; ++mi) {
    for (int rep = 0; rep < 2; ++rep) {
      CHECK_CUDA(cudaMemsetAsync(dstatus, 0, 16, stream));
      const int rc = sage_b200_sageattn(dq, dk, dv, dout, NULL, NULL, work, wbytes, dstatus, SAGE_B200_F16, B, Hq, Hkv, N, N, D,
                                        sq, sk, sk, sq, causal, sm_scale, blk_q, blk_k, warp_q, warp_k,
                                        SAGE_B200_GRAN_PER_THREAD, 1, modes[mi], SAGE_B200_DIV_FULL, stream);
      if (rc != SAGE_B200_OK) { fprintf(stderr, "sage_b200_sageattn failed: %d %s\n", rc, sage_b200_last_error()); return 1; }
      CHECK_CUDA(cudaMemcpyAsync(rep ? ho2 : ho, dout, nq * 2, cudaMemcpyDeviceToHost, stream));
      int32_t st[4];
      CHECK_CUDA(cudaMemcpyAsync(st, dstatus, 16, cudaMemcpyDeviceToHost, stream));
      CHECK_CUDA(cudaStreamSynchronize(stream));
      if (st[0] != 0) { fprintf(stderr, "kernel status %d\n", st[0]); return 1; }
    }
    if (memcmp(ho, ho2, nq * 2) != 0) { fprintf(stderr, "mode %d: two calls differ\n", modes[mi]); ++failures; }
    double num = 0.0, den = 0.0, max_abs = 0.0;
    for (size_t i = 0; i < nq; ++i) {
      const double d = (double)h2f(ho[i]) - (double)ref[i];
      num += d * d; den += (double)ref[i] * (double)ref[i];
      if (fabs(d) > max_abs) max_abs = fabs(d);
    }
    const double fro = sqrt(num / den);
    printf("pv_accum %d: fro_rel %.5f max_abs %.5f\n", modes[mi], fro, max_abs);
    if (!(fro <= 0.02 && max_abs <= 0.1)) ++failures;      /* the reference's own acceptance bounds (tests/test_sageattn.py:59) */
  }
  /* a bad argument comes back as an error code with a message, not as a crash */
  if (sage_b200_sageattn(dq, dk, dv, dout, NULL, NULL, work, 16, dstatus, SAGE_B200_F16, B, Hq, Hkv, N, N, D, sq, sk, sk, sq,
                         causal, sm_scale, blk_q, blk_k, warp_q, warp_k, SAGE_B200_GRAN_PER_THREAD, 1, SAGE_B200_PV_F32,
                         SAGE_B200_DIV_FULL, stream) == SAGE_B200_OK || strlen(sage_b200_last_error()) == 0) {
    fprintf(stderr, "a too-small workspace was accepted\n");
    ++failures;
  }
  printf(failures ? "FAIL\n" : "PASS\n");
  return failures ? 1 : 0;
}
