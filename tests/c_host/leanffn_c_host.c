/* A host written in plain C that drives the kernels through the C ABI alone (no Python, no torch): LayerNorm forward,
 * a GEMM with bias, the column sum with library-resident scratch, and a dropout mask, each checked against loops on
 * the host.  Built and run by tests/test_c_host.py; prints "C HOST OK" and exits 0 on success. */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "leanffn_b200.h"

#define CHECK_CUDA(call)                                                                   \
  do {                                                                                     \
    cudaError_t e_ = (call);                                                               \
    if (e_ != cudaSuccess) {                                                               \
      fprintf(stderr, "%s:%d cuda error %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
      return 2;                                                                            \
    }                                                                                      \
  } while (0)
#define CHECK_LEAN(call)                                                                        \
  do {                                                                                          \
    int32_t s_ = (call);                                                                        \
    if (s_ != LEANFFN_OK) {                                                                     \
      fprintf(stderr, "%s:%d leanffn status %d: %s\n", __FILE__, __LINE__, s_, leanffn_status_string(s_)); \
      return 3;                                                                                 \
    }                                                                                           \
  } while (0)

static float frand(uint32_t* state) { /* xorshift, uniform in [-1, 1) */
  uint32_t x = *state;
  x ^= x << 13, x ^= x >> 17, x ^= x << 5;
  *state = x;
  return (float)(x >> 8) / 8388608.0f - 1.0f;
}

static int close_enough(const float* got, const double* want, size_t n, double tol, const char* what) {
  double worst = 0.0;
  for (size_t i = 0; i < n; ++i) {
    const double err = fabs((double)got[i] - want[i]) / (1.0 + fabs(want[i]));
    if (!(err <= worst)) worst = err;
  }
  printf("%-28s max scaled error %.3g\n", what, worst);
  return worst <= tol;
}

int main(void) {
  enum { ROWS = 96, COLS = 200, OUT = 72 };
  uint32_t rng = 12345u;
  if (leanffn_abi_version() != LEANFFN_ABI_VERSION) return 1;

  float *x = malloc(sizeof(float) * ROWS * COLS), *w = malloc(sizeof(float) * OUT * COLS);
  float *gamma = malloc(sizeof(float) * COLS), *beta = malloc(sizeof(float) * COLS), *bias = malloc(sizeof(float) * OUT);
  for (int i = 0; i < ROWS * COLS; ++i) x[i] = 3.0f * frand(&rng) + 0.5f;
  for (int i = 0; i < OUT * COLS; ++i) w[i] = 0.1f * frand(&rng);
  for (int i = 0; i < COLS; ++i) gamma[i] = 1.0f + 0.1f * frand(&rng), beta[i] = 0.1f * frand(&rng);
  for (int i = 0; i < OUT; ++i) bias[i] = frand(&rng);

  float *dx, *dw, *dgamma, *dbeta, *dbias, *dy, *dout, *dsum;
  uint8_t* dmask;
  int32_t* dstatus;
  CHECK_CUDA(cudaMalloc((void**)&dx, sizeof(float) * ROWS * COLS));
  CHECK_CUDA(cudaMalloc((void**)&dy, sizeof(float) * ROWS * COLS));
  CHECK_CUDA(cudaMalloc((void**)&dw, sizeof(float) * OUT * COLS));
  CHECK_CUDA(cudaMalloc((void**)&dgamma, sizeof(float) * COLS));
  CHECK_CUDA(cudaMalloc((void**)&dbeta, sizeof(float) * COLS));
  CHECK_CUDA(cudaMalloc((void**)&dbias, sizeof(float) * OUT));
  CHECK_CUDA(cudaMalloc((void**)&dout, sizeof(float) * ROWS * OUT));
  CHECK_CUDA(cudaMalloc((void**)&dsum, sizeof(float) * OUT));
  CHECK_CUDA(cudaMalloc((void**)&dmask, ROWS * OUT));
  CHECK_CUDA(cudaMalloc((void**)&dstatus, sizeof(int32_t)));
  CHECK_CUDA(cudaMemset(dstatus, 0, sizeof(int32_t)));
  CHECK_CUDA(cudaMemcpy(dx, x, sizeof(float) * ROWS * COLS, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dw, w, sizeof(float) * OUT * COLS, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dgamma, gamma, sizeof(float) * COLS, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dbeta, beta, sizeof(float) * COLS, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dbias, bias, sizeof(float) * OUT, cudaMemcpyHostToDevice));
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));

  /* y = LayerNorm(x); out = y . W^T + bias; sums = column sums of out; mask = dropout keep flags */
  const float eps = 1e-5f;
  CHECK_LEAN(leanffn_layer_norm_forward(dx, LEANFFN_F32, dgamma, dbeta, LEANFFN_F32, dy, LEANFFN_F32, ROWS, COLS, eps,
                                        0.0f, 0, 0, NULL, 0, stream));
  leanffn_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.M = ROWS, d.N = OUT, d.K = COLS;
  d.in_dtype = LEANFFN_F32;
  d.A = dy, d.lda = COLS;
  d.B = dw, d.ldb = COLS;
  d.epilogue = LEANFFN_EPI_STORE;
  d.D = dout, d.ldd = OUT, d.d_dtype = LEANFFN_F32;
  d.bias = dbias, d.bias_dtype = LEANFFN_F32;
  d.status_word = dstatus;
  CHECK_LEAN(leanffn_gemm(&d, stream));
  if (leanffn_column_sum_static_capacity() < OUT) return 4;
  CHECK_LEAN(leanffn_column_sum_static(dout, LEANFFN_F32, OUT, dsum, ROWS, OUT, stream));
  CHECK_LEAN(leanffn_dropout_mask(dmask, ROWS * OUT, 0.25f, 7, 0, stream));
  CHECK_CUDA(cudaStreamSynchronize(stream));

  float *y = malloc(sizeof(float) * ROWS * COLS), *out = malloc(sizeof(float) * ROWS * OUT), sums[OUT];
  uint8_t* mask = malloc(ROWS * OUT);
  int32_t status = -1;
  CHECK_CUDA(cudaMemcpy(y, dy, sizeof(float) * ROWS * COLS, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(out, dout, sizeof(float) * ROWS * OUT, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(sums, dsum, sizeof(float) * OUT, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(mask, dmask, ROWS * OUT, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(&status, dstatus, sizeof(int32_t), cudaMemcpyDeviceToHost));
  if (status != LEANFFN_DEV_OK) return 5;

  double *y_ref = malloc(sizeof(double) * ROWS * COLS), *out_ref = malloc(sizeof(double) * ROWS * OUT), sum_ref[OUT];
  for (int r = 0; r < ROWS; ++r) {
    double mean = 0.0, var = 0.0;
    for (int c = 0; c < COLS; ++c) mean += x[r * COLS + c];
    mean /= COLS;
    for (int c = 0; c < COLS; ++c) var += (x[r * COLS + c] - mean) * (x[r * COLS + c] - mean);
    var /= COLS;
    for (int c = 0; c < COLS; ++c) y_ref[r * COLS + c] = (x[r * COLS + c] - mean) / sqrt(var + eps) * gamma[c] + beta[c];
  }
  for (int o = 0; o < OUT; ++o) sum_ref[o] = 0.0;
  for (int r = 0; r < ROWS; ++r)
    for (int o = 0; o < OUT; ++o) {
      double acc = bias[o];
      for (int c = 0; c < COLS; ++c) acc += y_ref[r * COLS + c] * w[o * COLS + c];
      out_ref[r * OUT + o] = acc;
      sum_ref[o] += acc;
    }
  int kept = 0;
  for (int i = 0; i < ROWS * OUT; ++i) kept += mask[i] != 0;
  const double keep_rate = (double)kept / (ROWS * OUT);
  printf("%-28s %.3f (expected 0.75)\n", "dropout keep rate", keep_rate);

  int ok = close_enough(y, y_ref, ROWS * COLS, 1e-4, "layer norm forward");
  ok &= close_enough(out, out_ref, ROWS * OUT, 1e-4, "gemm + bias (fp32 path)");
  ok &= close_enough(sums, sum_ref, OUT, 1e-4, "column sum, static scratch");
  ok &= fabs(keep_rate - 0.75) < 0.03;
  /* rejected arguments come back as negative codes, nothing is launched */
  ok &= leanffn_gemm(NULL, stream) == LEANFFN_ERR_NULL;
  d.K = 0;
  ok &= leanffn_gemm(&d, stream) == LEANFFN_ERR_SHAPE;
  if (!ok) return 6;
  printf("C HOST OK\n");
  return 0;
}
