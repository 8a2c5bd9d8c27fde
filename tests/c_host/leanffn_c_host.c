/* A host written in plain C that drives the kernels through the C ABI alone (no Python, no torch): LayerNorm forward,
 * a GEMM with bias, the column sum with library-resident scratch, and a dropout mask, each checked against loops on
 * the host.  With a file name as its argument it also runs one whole LeanFFN step (leanffn_ffn_forward +
 * leanffn_ffn_backward) on the case stored in that file and compares the output and every gradient with the values
 * stored beside the inputs (tests/test_c_host.py writes the file from a golden vector the reference produced).
 * Built and run by tests/test_c_host.py; prints "C HOST OK" and exits 0 on success. */
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

/* ---- one LeanFFN step from a flat file ----------------------------------------------------------------------------
 * File: 10 int64 (magic 0x4C45414E, tokens, hidden, intermediate, gated, residual, seed, elem_offset, dropout in ppm,
 * 0), then float32 arrays: x, g [T*H]; ln_w, ln_b [H]; W1 [N1*H], b1 [N1]; W2 [H*I], b2 [H]; then the expected
 * out, grad_input [T*H]; grad ln_w, ln_b [H]; grad W1, b1, W2, b2. */
static float* read_floats(FILE* f, size_t n) {
  float* p = malloc(sizeof(float) * (n ? n : 1));
  if (p != NULL && fread(p, sizeof(float), n, f) != n) {
    free(p);
    return NULL;
  }
  return p;
}

static int matches(const float* got, const float* want, size_t n, const char* what) {
  /* The rule of the Python parity tests for bf16 products against an fp64 run: |got - want| <= 1e-2 * max(1, S) +
   * 2e-2 * max(|want|, S) with S = rms(want); rounding noise has tails, so up to 0.1 % of the elements (at least one)
   * may lie beyond the bound, none beyond 4 times the bound. */
  double ss = 0.0, worst = 0.0;
  size_t beyond = 0;
  for (size_t i = 0; i < n; ++i) ss += (double)want[i] * want[i];
  const double S = sqrt(ss / (n ? n : 1));
  for (size_t i = 0; i < n; ++i) {
    const double mag = fabs(want[i]) > S ? fabs(want[i]) : S;
    const double ratio = fabs((double)got[i] - want[i]) / (1e-2 * (S > 1.0 ? S : 1.0) + 2e-2 * mag);
    if (!(ratio <= worst)) worst = ratio;
    if (!(ratio <= 1.0)) ++beyond;
  }
  printf("%-28s worst error / bound %.3f, %zu of %zu beyond the bound\n", what, worst, beyond, n);
  return worst <= 4.0 && beyond <= 1 + n / 1000;
}

static int upload(void** dst, const float* src, size_t n) {
  if (cudaMalloc(dst, sizeof(float) * (n ? n : 1)) != cudaSuccess) return 0;
  return cudaMemcpy(*dst, src, sizeof(float) * n, cudaMemcpyHostToDevice) == cudaSuccess;
}

static int run_block_case(const char* path) {
  FILE* f = fopen(path, "rb");
  if (f == NULL) return 20;
  int64_t head[10];
  if (fread(head, sizeof(int64_t), 10, f) != 10 || head[0] != 0x4C45414E) return 21;
  const int64_t T = head[1], H = head[2], I = head[3], gated = head[4], residual = head[5];
  const int64_t N1 = gated ? 2 * I : I;
  const float p_drop = (float)head[8] * 1e-6f;
  const size_t sizes[16] = {T * H, T * H, H, H, N1 * H, N1, H * I, H, T * H, T * H, H, H, N1 * H, N1, H * I, H};
  float* h[16];
  for (int i = 0; i < 16; ++i)
    if ((h[i] = read_floats(f, sizes[i])) == NULL) return 22;
  fclose(f);

  void* dev[8]; /* x, g, ln_w, ln_b, W1 (fp32), b1, W2 (fp32), b2 */
  for (int i = 0; i < 8; ++i)
    if (!upload(&dev[i], h[i], sizes[i])) return 23;
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));
  /* weights enter the block in the compute type: bf16 copies made on the device */
  void *w1_bf16, *w2_bf16;
  CHECK_CUDA(cudaMalloc(&w1_bf16, 2 * sizes[4]));
  CHECK_CUDA(cudaMalloc(&w2_bf16, 2 * sizes[6]));
  CHECK_LEAN(leanffn_cast(dev[4], LEANFFN_F32, w1_bf16, LEANFFN_BF16, (int64_t)sizes[4], stream));
  CHECK_LEAN(leanffn_cast(dev[6], LEANFFN_F32, w2_bf16, LEANFFN_BF16, (int64_t)sizes[6], stream));
  int32_t* status;
  CHECK_CUDA(cudaMalloc((void**)&status, sizeof(int32_t)));
  CHECK_CUDA(cudaMemset(status, 0, sizeof(int32_t)));

  leanffn_ffn_desc d;
  memset(&d, 0, sizeof(d));
  d.tokens = T, d.hidden = (int32_t)H, d.intermediate = (int32_t)I;
  d.gated = (int32_t)gated, d.act = LEANFFN_ACT_GELU_TANH, d.residual = (int32_t)residual;
  d.compute_dtype = LEANFFN_BF16, d.io_dtype = LEANFFN_F32, d.grad_out_dtype = LEANFFN_F32, d.param_dtype = LEANFFN_F32;
  d.eps = 1e-12f, d.dropout_p = p_drop, d.seed = (uint64_t)head[6], d.elem_offset = (uint64_t)head[7];
  d.ln_weight = dev[2], d.ln_bias = dev[3];
  d.i2h.weight = w1_bf16, d.i2h.bias = dev[5], d.i2h.bias_dtype = LEANFFN_F32;
  d.h2o.weight = w2_bf16, d.h2o.bias = dev[7], d.h2o.bias_dtype = LEANFFN_F32;
  d.status_word = status;

  const size_t ws_f = leanffn_ffn_workspace_bytes(&d, 0), ws_b = leanffn_ffn_workspace_bytes(&d, 1);
  if (ws_f == 0 || ws_b == 0) return 24;
  void *workspace, *out_bf16, *pre;
  CHECK_CUDA(cudaMalloc(&workspace, ws_f > ws_b ? ws_f : ws_b));
  CHECK_CUDA(cudaMalloc(&out_bf16, 2 * sizes[0]));
  CHECK_CUDA(cudaMalloc(&pre, 2 * (size_t)(T * N1)));
  CHECK_LEAN(leanffn_ffn_forward(&d, dev[0], out_bf16, pre, NULL, NULL, workspace, stream));

  leanffn_ffn_grads grads;
  memset(&grads, 0, sizeof(grads));
  void* gdev[8]; /* out (fp32 copy), grad_input, ln_w, ln_b, W1, b1, W2, b2 */
  for (int i = 0; i < 8; ++i) CHECK_CUDA(cudaMalloc(&gdev[i], sizeof(float) * (sizes[8 + i] ? sizes[8 + i] : 1)));
  grads.grad_input = gdev[1], grads.grad_ln_weight = gdev[2], grads.grad_ln_bias = gdev[3];
  grads.grad_i2h_weight = gdev[4], grads.grad_i2h_bias = gdev[5];
  grads.grad_h2o_weight = gdev[6], grads.grad_h2o_bias = gdev[7];
  CHECK_LEAN(leanffn_ffn_backward(&d, dev[1], dev[0], pre, NULL, NULL, &grads, workspace, stream));
  CHECK_LEAN(leanffn_cast(out_bf16, LEANFFN_BF16, gdev[0], LEANFFN_F32, (int64_t)sizes[0], stream));
  CHECK_CUDA(cudaStreamSynchronize(stream));
  int32_t code = -1;
  CHECK_CUDA(cudaMemcpy(&code, status, sizeof(int32_t), cudaMemcpyDeviceToHost));
  if (code != LEANFFN_DEV_OK) return 25;

  static const char* names[8] = {"block: out", "block: grad_input", "block: grad ln weight", "block: grad ln bias",
                                 "block: grad W1", "block: grad b1", "block: grad W2", "block: grad b2"};
  int ok = 1;
  for (int i = 0; i < 8; ++i) {
    float* got = malloc(sizeof(float) * (sizes[8 + i] ? sizes[8 + i] : 1));
    CHECK_CUDA(cudaMemcpy(got, gdev[i], sizeof(float) * sizes[8 + i], cudaMemcpyDeviceToHost));
    ok &= matches(got, h[8 + i], sizes[8 + i], names[i]);
    free(got);
  }
  /* a rejected descriptor costs nothing: no workspace, a negative code */
  d.hidden = 31;
  ok &= leanffn_ffn_workspace_bytes(&d, 0) == 0;
  ok &= leanffn_ffn_forward(&d, dev[0], out_bf16, pre, NULL, NULL, workspace, stream) == LEANFFN_ERR_SHAPE;
  return ok ? 0 : 26;
}

/* ---- one attention-core step from a flat file ----------------------------------------------------------------------
 * File: 6 int64 (magic 0x4154544E, batch, len, heads, head_dim, 0), then float32 arrays: q, k, v, grad_out
 * [batch * len * hidden]; mask [batch * len * len] (additive, shared by the heads); then the expected out, grad_q,
 * grad_k, grad_v [batch * len * hidden] of the reference's SimpleAttentionCore. */
static int run_attention_case(const char* path) {
  FILE* f = fopen(path, "rb");
  if (f == NULL) return 30;
  int64_t head[6];
  if (fread(head, sizeof(int64_t), 6, f) != 6 || head[0] != 0x4154544E) return 31;
  const int64_t B = head[1], S = head[2], HEADS = head[3], D = head[4];
  const size_t n = (size_t)(B * S * HEADS * D), nm = (size_t)(B * S * S);
  const size_t sizes[9] = {n, n, n, n, nm, n, n, n, n};
  float* h[9];
  for (int i = 0; i < 9; ++i)
    if ((h[i] = read_floats(f, sizes[i])) == NULL) return 32;
  fclose(f);

  cudaStream_t stream;
  if (cudaStreamCreate(&stream) != cudaSuccess) return 33;
  void *f32[4], *b16[4], *mask, *out, *dk, *dv, *lse, *delta, *dq, *back;
  int32_t* status;
  for (int i = 0; i < 4; ++i) { /* q, k, v, grad_out: upload as fp32, convert to bf16 on the device */
    if (!upload(&f32[i], h[i], n) || cudaMalloc(&b16[i], 2 * n) != cudaSuccess) return 34;
    if (leanffn_cast(f32[i], LEANFFN_F32, b16[i], LEANFFN_BF16, (int64_t)n, stream) != LEANFFN_OK) return 35;
  }
  if (!upload(&mask, h[4], nm)) return 34;
  if (cudaMalloc(&out, 2 * n) != cudaSuccess || cudaMalloc(&dk, 2 * n) != cudaSuccess || cudaMalloc(&dv, 2 * n) != cudaSuccess ||
      cudaMalloc(&dq, 4 * n) != cudaSuccess || cudaMalloc(&back, 4 * n) != cudaSuccess ||
      cudaMalloc(&lse, 4 * (size_t)(B * HEADS * S)) != cudaSuccess || cudaMalloc(&delta, 4 * (size_t)(B * HEADS * S)) != cudaSuccess ||
      cudaMalloc((void**)&status, sizeof(int32_t)) != cudaSuccess || cudaMemset(status, 0, sizeof(int32_t)) != cudaSuccess)
    return 34;

  leanffn_attention_desc d;
  memset(&d, 0, sizeof(d));
  d.batch = (int32_t)B, d.heads = (int32_t)HEADS, d.q_len = (int32_t)S, d.kv_len = (int32_t)S, d.head_dim = (int32_t)D;
  d.scale = 1.0f / sqrtf((float)D);
  d.q = b16[0], d.k = b16[1], d.v = b16[2];
  d.ld_q = d.ld_k = d.ld_v = HEADS * D;
  d.mask = (const float*)mask, d.mask_stride_b = S * S, d.mask_stride_h = 0, d.mask_stride_q = S;
  d.out = out, d.ld_out = HEADS * D, d.lse = (float*)lse;
  d.d_out = b16[3], d.ld_dout = HEADS * D, d.delta = (float*)delta, d.dq_accum = (float*)dq;
  d.dk = dk, d.dv = dv, d.ld_dk = d.ld_dv = HEADS * D;
  d.status_word = status;
  if (leanffn_attention_forward(&d, stream) != LEANFFN_OK) return 36;
  if (leanffn_attention_backward(&d, stream) != LEANFFN_OK) return 37;
  float* got = malloc(sizeof(float) * n);
  int32_t word = -1;
  int ok = got != NULL;
  void* results[3] = {out, dk, dv};
  const int expected[3] = {5, 7, 8};
  const char* names[3] = {"attention: out", "attention: grad k", "attention: grad v"};
  for (int i = 0; ok && i < 3; ++i) { /* bf16 results come back through the cast kernel */
    ok &= leanffn_cast(results[i], LEANFFN_BF16, back, LEANFFN_F32, (int64_t)n, stream) == LEANFFN_OK;
    ok &= cudaMemcpyAsync(got, back, 4 * n, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
    ok &= cudaStreamSynchronize(stream) == cudaSuccess;
    ok &= matches(got, h[expected[i]], n, names[i]);
  }
  ok &= cudaMemcpy(got, dq, 4 * n, cudaMemcpyDeviceToHost) == cudaSuccess && matches(got, h[6], n, "attention: grad q");
  ok &= cudaMemcpy(&word, status, sizeof(word), cudaMemcpyDeviceToHost) == cudaSuccess && word == 0;
  /* rejected arguments: a head size the kernels do not take, a missing output */
  d.head_dim = 24;
  ok &= leanffn_attention_forward(&d, stream) == LEANFFN_ERR_UNSUPPORTED;
  d.head_dim = (int32_t)D, d.out = NULL;
  ok &= leanffn_attention_forward(&d, stream) == LEANFFN_ERR_NULL;
  return ok ? 0 : 38;
}

int main(int argc, char** argv) {
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
  if (argc > 1) {
    const int code = run_block_case(argv[1]);
    if (code != 0) {
      fprintf(stderr, "whole-block step failed with code %d\n", code);
      return code;
    }
  }
  if (argc > 2) {
    const int code = run_attention_case(argv[2]);
    if (code != 0) {
      fprintf(stderr, "attention step failed with code %d\n", code);
      return code;
    }
  }
  printf("C HOST OK\n");
  return 0;
}
