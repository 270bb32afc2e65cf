/* A host written in plain C against include/ffnk.h: no Python, no torch, no C++.
 *
 * It does what a maintainer's FFI binding would do (cudaMalloc'd buffers, the default stream, the
 * entry points in the order the header describes) on one small problem and checks the results
 * against a float loop over the same bf16-rounded inputs:
 *   routing lists bit for bit, MaskedLinear forward and the whole MaskedFFN forward to 1e-2 of the
 *   output's maximum (the tolerance of the Python parity tests).
 * Prints "cabi_host: OK" and returns 0, or says what differed and returns 1.
 *
 * Built by ffn_kernel_b200/build.py (gcc + libcudart + libffnk.so); run by tests/test_gpu_cabi_host.py.
 */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ffnk.h"

#define CHECK_CUDA(x)                                                                      \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      fprintf(stderr, "cabi_host: %s -> %s\n", #x, cudaGetErrorString(e_));                \
      return 1;                                                                            \
    }                                                                                      \
  } while (0)

#define CHECK_FFNK(x)                                                                      \
  do {                                                                                     \
    int r_ = (x);                                                                          \
    if (r_ != 0) {                                                                         \
      fprintf(stderr, "cabi_host: %s -> %d (%s)\n", #x, r_, ffnk_status_string(r_));       \
      return 1;                                                                            \
    }                                                                                      \
  } while (0)

static uint32_t lcg_state = 12345u;
static float lcg_uniform(void) { /* (-1, 1) */
  lcg_state = lcg_state * 1664525u + 1013904223u;
  return (float)((lcg_state >> 8) & 0xFFFFFF) / 8388608.0f - 1.0f;
}

static uint16_t f32_to_bf16(float f) { /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static void fill(uint16_t* dst, float* as_float, size_t n, float scale) {
  for (size_t i = 0; i < n; ++i) {
    dst[i] = f32_to_bf16(lcg_uniform() * scale);
    as_float[i] = bf16_to_f32(dst[i]);
  }
}

static float silu(float v) { return v / (1.0f + expf(-v)); }

/* max |got - want| / max |want| */
static double max_rel_err(const uint16_t* got, const float* want, size_t n) {
  double num = 0.0, den = 0.0;
  for (size_t i = 0; i < n; ++i) {
    double d = fabs((double)bf16_to_f32(got[i]) - (double)want[i]);
    if (d > num) num = d;
    if (fabs((double)want[i]) > den) den = fabs((double)want[i]);
  }
  return den > 0.0 ? num / den : num;
}

int main(void) {
  enum { M = 333, D = 72, H = 136 }; /* rows not a multiple of 128, widths multiples of 8 only */
  const int64_t cap = ffnk_route_capacity(M);
  if (ffnk_version() < 100 || cap < M || cap % 128) {
    fprintf(stderr, "cabi_host: unexpected version or capacity\n");
    return 1;
  }

  /* ---------------- host data: nn.Linear storage [out, in], handed over as the [in, out] view */
  static uint16_t x16[M * D], w16[6][H * D];
  static float xf[M * D], wf[6][H * D];
  static uint8_t mask[M];
  fill(x16, xf, (size_t)M * D, 1.0f);
  for (int i = 0; i < 6; ++i) fill(w16[i], wf[i], (size_t)H * D, 0.1f);
  for (int m = 0; m < M; ++m) mask[m] = (uint8_t)(((m / 7) % 3) != 0); /* runs of 7 and 14 tokens */
  /* w[0] = W1 [H, D], w[1] = W2 [D, H], w[2] = W3 [H, D]; w[3..5] = U1, U2, U3 the same way */

  /* ---------------- device buffers */
  void *dx, *dw[6], *dmask, *dperm, *dcounts, *dscan, *dstatus, *dws, *dy, *dlin;
  const int64_t ws_bytes = ffnk_ffn_workspace_bytes(M, D, H);
  CHECK_CUDA(cudaMalloc(&dx, sizeof x16));
  for (int i = 0; i < 6; ++i) CHECK_CUDA(cudaMalloc(&dw[i], sizeof w16[i]));
  CHECK_CUDA(cudaMalloc(&dmask, M));
  CHECK_CUDA(cudaMalloc(&dperm, (size_t)(2 * cap) * 4));
  CHECK_CUDA(cudaMalloc(&dcounts, 8 * 4));
  CHECK_CUDA(cudaMalloc(&dscan, (size_t)ffnk_route_workspace_bytes(M)));
  CHECK_CUDA(cudaMalloc(&dstatus, 4));
  CHECK_CUDA(cudaMalloc(&dws, (size_t)ws_bytes));
  CHECK_CUDA(cudaMalloc(&dy, (size_t)M * D * 2));
  CHECK_CUDA(cudaMalloc(&dlin, (size_t)M * H * 2));
  CHECK_CUDA(cudaMemset(dstatus, 0, 4));
  CHECK_CUDA(cudaMemcpy(dx, x16, sizeof x16, cudaMemcpyHostToDevice));
  for (int i = 0; i < 6; ++i) CHECK_CUDA(cudaMemcpy(dw[i], w16[i], sizeof w16[i], cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dmask, mask, M, cudaMemcpyHostToDevice));

  /* ---------------- routing: bit-exact lists */
  CHECK_FFNK(ffnk_route(dmask, M, (int32_t*)dperm, (int32_t*)dcounts, dscan, (int32_t*)dstatus, NULL));
  static int32_t perm[2 * 512], counts[8];
  CHECK_CUDA(cudaMemcpy(perm, dperm, (size_t)(2 * cap) * 4, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(counts, dcounts, sizeof counts, cudaMemcpyDeviceToHost));
  int mv = 0, mt = 0, runs = 0;
  for (int m = 0; m < M; ++m) {
    if (m == 0 || (mask[m] != 0) != (mask[m - 1] != 0)) ++runs;
    if (mask[m]) {
      if (perm[mv] != m) { fprintf(stderr, "cabi_host: visual list differs at %d\n", mv); return 1; }
      ++mv;
    } else {
      if (perm[cap + mt] != m) { fprintf(stderr, "cabi_host: text list differs at %d\n", mt); return 1; }
      ++mt;
    }
  }
  if (counts[0] != mv || counts[1] != mt || counts[2] != cap || counts[3] != M || counts[4] != runs) {
    fprintf(stderr, "cabi_host: counts differ: %d %d %d %d %d\n", counts[0], counts[1], counts[2], counts[3], counts[4]);
    return 1;
  }

  /* ---------------- MaskedLinear forward: lin[m] = x[m] @ (mask ? W1 : U1)^T, weights as the .T view */
  CHECK_FFNK(ffnk_linear_fwd(dx, D, dw[0], dw[3], /*stride_k*/ 1, /*stride_n*/ D, (int32_t*)dperm, (int32_t*)dcounts, dlin,
                             H, NULL, M, H, D, (int32_t*)dstatus, NULL));
  /* ---------------- MaskedFFN forward in one call */
  CHECK_FFNK(ffnk_ffn_forward(dx, D, dw[0], dw[1], dw[2], dw[3], dw[4], dw[5], 1, D, 1, H, dmask, dws, ws_bytes, dy, D, M,
                              D, H, /*allow_decode*/ 1, (int32_t*)dstatus, NULL));
  CHECK_FFNK(ffnk_read_status((int32_t*)dstatus, 1, NULL));

  static uint16_t lin16[M * H], y16[M * D];
  CHECK_CUDA(cudaMemcpy(lin16, dlin, sizeof lin16, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(y16, dy, sizeof y16, cudaMemcpyDeviceToHost));

  /* ---------------- float reference on the bf16-rounded inputs */
  static float lin_ref[M * H], y_ref[M * D], hid[H];
  for (int m = 0; m < M; ++m) {
    const int o = mask[m] ? 0 : 3;
    for (int j = 0; j < H; ++j) {
      float t1 = 0.f, t3 = 0.f;
      for (int k = 0; k < D; ++k) {
        t1 += xf[m * D + k] * wf[o][j * D + k];
        t3 += xf[m * D + k] * wf[o + 2][j * D + k];
      }
      lin_ref[m * H + j] = t1;
      hid[j] = silu(t1) * t3;
    }
    for (int c = 0; c < D; ++c) {
      float acc = 0.f;
      for (int j = 0; j < H; ++j) acc += hid[j] * wf[o + 1][c * H + j];
      y_ref[m * D + c] = acc;
    }
  }
  /* ---------------- training forward: counts is int32[8] (as for ffnk_route); the word behind it must stay untouched,
   * and y must equal the inference forward's y bit for bit */
  {
    const size_t rows = (size_t)cap + 512;
    void *tcounts, *txr, *tt1, *tt3, *thid, *ty;
    static int32_t guard_in[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0x5EED5EED}, guard_out[9];
    static uint16_t y_train[M * D];
    CHECK_CUDA(cudaMalloc(&tcounts, sizeof guard_in));
    CHECK_CUDA(cudaMemcpy(tcounts, guard_in, sizeof guard_in, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMalloc(&txr, rows * D * 2));
    CHECK_CUDA(cudaMalloc(&tt1, rows * H * 2));
    CHECK_CUDA(cudaMalloc(&tt3, rows * H * 2));
    CHECK_CUDA(cudaMalloc(&thid, rows * H * 2));
    CHECK_CUDA(cudaMalloc(&ty, (size_t)M * D * 2));
    CHECK_FFNK(ffnk_ffn_forward_train(dx, D, dw[0], dw[1], dw[2], dw[3], dw[4], dw[5], 1, D, 1, H, dmask, (int32_t*)dperm,
                                      (int32_t*)tcounts, dscan, txr, tt1, tt3, thid, ty, D, M, D, H, (int32_t*)dstatus,
                                      NULL));
    CHECK_FFNK(ffnk_read_status((int32_t*)dstatus, 1, NULL));
    CHECK_CUDA(cudaMemcpy(guard_out, tcounts, sizeof guard_out, cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(y_train, ty, sizeof y_train, cudaMemcpyDeviceToHost));
    if (guard_out[8] != 0x5EED5EED || guard_out[0] != mv || guard_out[1] != mt || guard_out[4] != runs) {
      fprintf(stderr, "cabi_host: training forward wrote outside counts[8] or wrong counts (guard %x)\n", guard_out[8]);
      return 1;
    }
    if (memcmp(y_train, y16, sizeof y16) != 0) {
      fprintf(stderr, "cabi_host: training forward and inference forward disagree\n");
      return 1;
    }
  }

  const double e_lin = max_rel_err(lin16, lin_ref, (size_t)M * H);
  const double e_ffn = max_rel_err(y16, y_ref, (size_t)M * D);
  printf("cabi_host: routing exact (Mv=%d Mt=%d runs=%d), linear %.2e, ffn %.2e\n", mv, mt, runs, e_lin, e_ffn);
  if (!(e_lin < 1e-2) || !(e_ffn < 1e-2)) {
    fprintf(stderr, "cabi_host: outside the 1e-2 tolerance\n");
    return 1;
  }
  puts("cabi_host: OK");
  return 0;
}
