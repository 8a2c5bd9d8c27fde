// Whole-block entry points: one call runs the forward (or the backward) schedule of a LeanFFN block on the caller's
// stream, out of caller-owned buffers.  The schedule is the reference's (lean_transformer/ffn.py:146-217 forward,
// :220-306 backward): pre-LayerNorm -> input projection (+ low rank) with the (gated) activation in its epilogue ->
// output projection with bias + dropout + residual in its epilogue; the backward rematerialises the activation and
// the LayerNorm output, keeps the bias gradients inside the kernels that produce their operands, and returns
// gradients for every parameter.  Everything is a launch of this library's own kernels through the same entry
// points a piecewise caller would use (leanffn_gemm, leanffn_layer_norm_*, ...); nothing is allocated or synchronised.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "gemm_common.cuh"
#include "nvtx_range.cuh"

using namespace leanffn;

namespace {

constexpr size_t ALIGN = 256;
inline size_t up(size_t n) { return (n + ALIGN - 1) / ALIGN * ALIGN; }

struct Carver {
  char* base;
  size_t used;
  void* take(size_t bytes) {
    void* p = base == nullptr ? nullptr : base + used;
    used += up(bytes);
    return p;
  }
};

struct FwdPlan {
  void *xhat, *hid;
  size_t bytes;
};
struct BwdPlan {
  void *dyp, *dres, *dpre, *hid, *xhat, *dxhat, *glr1, *glr2;
  float* partial;
  void* scratch;
  size_t bytes;
};

inline int64_t width1(const leanffn_ffn_desc* d) { return d->gated ? 2 * static_cast<int64_t>(d->intermediate) : d->intermediate; }

int32_t validate(const leanffn_ffn_desc* d) {
  if (d == nullptr) return LEANFFN_ERR_NULL;
  if (d->tokens < 0 || d->tokens > 0x7fffffff || d->hidden <= 0 || d->intermediate <= 0) return LEANFFN_ERR_SHAPE;
  if (d->compute_dtype != LEANFFN_BF16) return LEANFFN_ERR_UNSUPPORTED;  // fp32 mode is driven piecewise by the caller
  if (d->io_dtype != LEANFFN_F32 && d->io_dtype != LEANFFN_BF16) return LEANFFN_ERR_DTYPE;
  if (d->grad_out_dtype != LEANFFN_F32 && d->grad_out_dtype != LEANFFN_BF16) return LEANFFN_ERR_DTYPE;
  if (d->param_dtype != LEANFFN_F32 && d->param_dtype != LEANFFN_BF16) return LEANFFN_ERR_DTYPE;
  if (d->io_dtype == LEANFFN_F32 && d->param_dtype == LEANFFN_BF16) return LEANFFN_ERR_DTYPE;  // no such LayerNorm kernel
  if (d->act < 0 || d->act >= LEANFFN_ACT_COUNT) return LEANFFN_ERR_UNSUPPORTED;
  if (!(d->dropout_p >= 0.f && d->dropout_p < 1.f)) return LEANFFN_ERR_UNSUPPORTED;
  if (d->hidden % 8 != 0 || d->intermediate % 8 != 0) return LEANFFN_ERR_SHAPE;  // 16-byte rows for the tensor-core path
  for (const leanffn_linear_desc* l : {&d->i2h, &d->h2o}) {
    if (l->weight == nullptr) return LEANFFN_ERR_NULL;
    if (l->rank < 0 || (l->rank > 0 && (l->lowrank_first == nullptr || l->lowrank_second == nullptr))) return LEANFFN_ERR_NULL;
    if (l->rank % 8 != 0) return LEANFFN_ERR_SHAPE;
    if (l->bs_block < 0) return LEANFFN_ERR_SHAPE;
    if (l->bs_block > 0 && (l->fwd_index == nullptr || l->dgrad_index == nullptr || l->wgrad_index == nullptr ||
                            l->bs_num_blocks <= 0 || l->fwd_nnz <= 0 || l->dgrad_nnz <= 0))
      return LEANFFN_ERR_NULL;
  }
  return LEANFFN_OK;
}

FwdPlan plan_forward(const leanffn_ffn_desc* d, void* ws) {
  Carver c{static_cast<char*>(ws), 0};
  FwdPlan p{};
  const size_t T = static_cast<size_t>(d->tokens);
  p.xhat = c.take(T * d->hidden * 2);
  p.hid = c.take(T * d->intermediate * 2);
  p.bytes = c.used;
  return p;
}

size_t max3(size_t a, size_t b, size_t c) { return a > b ? (a > c ? a : c) : (b > c ? b : c); }

BwdPlan plan_backward(const leanffn_ffn_desc* d, void* ws) {
  Carver c{static_cast<char*>(ws), 0};
  BwdPlan p{};
  const size_t T = static_cast<size_t>(d->tokens);
  const size_t H = d->hidden, I = d->intermediate, N1 = static_cast<size_t>(width1(d));
  const bool recast = d->grad_out_dtype != LEANFFN_BF16;
  p.dyp = (d->dropout_p > 0.f || recast) ? c.take(T * H * 2) : nullptr;
  p.dres = (d->residual && recast) ? c.take(T * H * 2) : nullptr;
  p.dpre = c.take(T * N1 * 2);
  p.hid = c.take(T * I * 2);
  p.xhat = c.take(T * H * 2);
  p.dxhat = c.take(T * H * 2);
  p.glr1 = d->i2h.rank > 0 ? c.take(T * d->i2h.rank * 2) : nullptr;
  p.glr2 = d->h2o.rank > 0 ? c.take(T * d->h2o.rank * 2) : nullptr;
  p.partial = static_cast<float*>(c.take(((T + 31) / 32) * N1 * 4));
  const size_t s1 = leanffn_dropout_colsum_scratch_bytes(d->tokens, d->hidden);
  const size_t s2 = leanffn_column_sum_scratch_bytes((d->tokens + 31) / 32, static_cast<int64_t>(N1));
  const size_t s3 = leanffn_layer_norm_backward_scratch_bytes(d->tokens, d->hidden);
  p.scratch = c.take(max3(s1, s2, s3) + 16);
  p.bytes = c.used;
  return p;
}

// ---- product helpers -------------------------------------------------------------------------------------------
void base_desc(const leanffn_ffn_desc* d, leanffn_gemm_desc* g) {
  memset(g, 0, sizeof(*g));
  g->in_dtype = LEANFFN_BF16;
  g->d_dtype = LEANFFN_BF16;
  g->status_word = d->status_word;
  g->max_ctas = d->max_ctas;
  g->wait_limit_cycles = 0;
  g->timer = d->timer;
}

// D[M, N] = A[M, K] . B^T with B either [N, K] (b_mn = 0) or [K, N] (b_mn = 1), dense operands, plain store
int32_t plain_product(const leanffn_ffn_desc* d, const void* A, int64_t lda, bool a_mn, const void* B, int64_t ldb,
                      bool b_mn, int64_t M, int64_t N, int64_t K, void* D, int64_t ldd, int32_t d_dtype, cudaStream_t st) {
  leanffn_gemm_desc g;
  base_desc(d, &g);
  g.M = static_cast<int32_t>(M), g.N = static_cast<int32_t>(N), g.K = static_cast<int32_t>(K);
  g.A = A, g.lda = lda, g.a_mn_major = a_mn;
  g.B = B, g.ldb = ldb, g.b_mn_major = b_mn;
  g.D = D, g.ldd = ldd, g.d_dtype = d_dtype;
  return leanffn_gemm(&g, st);
}

// forward product of one projection: x [T, in] . W^T (+ low rank) with the given epilogue fields already in g
int32_t forward_product(const leanffn_ffn_desc* d, const leanffn_linear_desc* l, leanffn_gemm_desc* g, const void* x,
                        int64_t in_features, int64_t out_features, const void* lowrank_hid, cudaStream_t st) {
  g->M = static_cast<int32_t>(d->tokens), g->N = static_cast<int32_t>(out_features), g->K = static_cast<int32_t>(in_features);
  g->A = x, g->lda = in_features;
  g->B = l->weight;
  if (l->bs_block > 0) {
    g->bs_mode = 1, g->bs_block = l->bs_block, g->bs_nnz = l->fwd_nnz, g->bs_num_blocks = l->bs_num_blocks;
    g->bs_index = l->fwd_index, g->bs_count = l->fwd_count;
    g->ldb = l->bs_block;
  } else {
    g->ldb = in_features;
  }
  if (l->rank > 0) {
    g->A2 = lowrank_hid, g->lda2 = l->rank;
    g->B2 = l->lowrank_second, g->ldb2 = l->rank;
    g->K2 = l->rank;
  }
  g->bias = l->bias, g->bias_dtype = l->bias_dtype;
  return leanffn_gemm(g, st);
}

// input gradient of one projection: dy [T, out] . W (+ low-rank continuation) with the epilogue fields already in g
int32_t input_grad_product(const leanffn_ffn_desc* d, const leanffn_linear_desc* l, leanffn_gemm_desc* g, const void* dy,
                           int64_t in_features, int64_t out_features, const void* grad_lowrank_hid, cudaStream_t st) {
  g->M = static_cast<int32_t>(d->tokens), g->N = static_cast<int32_t>(in_features), g->K = static_cast<int32_t>(out_features);
  g->A = dy, g->lda = out_features;
  g->B = l->weight, g->b_mn_major = 1;
  if (l->bs_block > 0) {
    g->bs_mode = 2, g->bs_block = l->bs_block, g->bs_nnz = l->dgrad_nnz, g->bs_num_blocks = l->bs_num_blocks;
    g->bs_index = l->dgrad_index, g->bs_count = l->dgrad_count;
    g->ldb = l->bs_block;
  } else {
    g->ldb = in_features;
  }
  if (l->rank > 0) {
    g->A2 = grad_lowrank_hid, g->lda2 = l->rank;
    g->B2 = l->lowrank_first, g->ldb2 = in_features;  // [rank, in] read MN-major: K2 = rank rows of N = in columns
    g->K2 = l->rank;
  }
  return leanffn_gemm(g, st);
}

// weight gradient of one projection in the weight's own storage format: dy^T . x
int32_t weight_grad_product(const leanffn_ffn_desc* d, const leanffn_linear_desc* l, const void* dy, const void* x,
                            int64_t in_features, int64_t out_features, void* dw, int32_t dw_dtype, cudaStream_t st) {
  leanffn_gemm_desc g;
  base_desc(d, &g);
  g.a_mn_major = g.b_mn_major = 1;
  g.A = dy, g.lda = out_features;
  g.B = x, g.ldb = in_features;
  g.K = static_cast<int32_t>(d->tokens);
  g.D = dw, g.d_dtype = dw_dtype;
  if (l->bs_block > 0) {
    g.bs_mode = 3, g.bs_block = l->bs_block, g.bs_nnz = 1, g.bs_num_blocks = l->bs_num_blocks;
    g.bs_index = l->wgrad_index;
    g.bs_wgrad_pairs = l->wgrad_pairs;
    g.M = l->bs_num_blocks * l->bs_block, g.N = l->bs_block, g.ldd = l->bs_block;
  } else {
    g.M = static_cast<int32_t>(out_features), g.N = static_cast<int32_t>(in_features), g.ldd = in_features;
  }
  return leanffn_gemm(&g, st);
}

#define RUN(call)                        \
  do {                                   \
    const int32_t s_ = (call);           \
    if (s_ != LEANFFN_OK) return s_;     \
  } while (0)

}  // namespace

extern "C" size_t leanffn_ffn_workspace_bytes(const leanffn_ffn_desc* d, int32_t backward) {
  if (validate(d) != LEANFFN_OK) return 0;
  return (backward ? plan_backward(d, nullptr).bytes : plan_forward(d, nullptr).bytes) + ALIGN;
}

extern "C" int32_t leanffn_ffn_forward(const leanffn_ffn_desc* d, const void* x, void* out, void* pre_activation,
                                       void* i2h_lowrank_hid, void* h2o_lowrank_hid, void* workspace, void* stream) {
  NvtxRange range("leanffn_ffn_forward");
  RUN(validate(d));
  if (d->tokens == 0) return LEANFFN_OK;
  if (x == nullptr || out == nullptr || pre_activation == nullptr || workspace == nullptr) return LEANFFN_ERR_NULL;
  if ((d->i2h.rank > 0 && i2h_lowrank_hid == nullptr) || (d->h2o.rank > 0 && h2o_lowrank_hid == nullptr)) return LEANFFN_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) % ALIGN != 0) return LEANFFN_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const FwdPlan p = plan_forward(d, workspace);
  const int64_t T = d->tokens, H = d->hidden, I = d->intermediate, N1 = width1(d);

  // pre-LayerNorm: lean_transformer/ffn.py:184
  RUN(leanffn_layer_norm_forward(x, d->io_dtype, d->ln_weight, d->ln_bias, d->param_dtype, p.xhat, LEANFFN_BF16, T, H, d->eps,
                                 0.f, 0, 0, nullptr, 0, st));
  // input projection (+ low rank) with the activation in its epilogue: ffn.py:185-189, linear.py:207-230
  if (d->i2h.rank > 0)
    RUN(plain_product(d, p.xhat, H, false, d->i2h.lowrank_first, H, false, T, d->i2h.rank, H, i2h_lowrank_hid, d->i2h.rank,
                      LEANFFN_BF16, st));
  {
    leanffn_gemm_desc g;
    base_desc(d, &g);
    const bool fuse = d->i2h.bs_block == 0 || (d->gated && d->i2h.fuse_gated_forward);
    g.D = pre_activation, g.ldd = N1;
    if (fuse) {
      g.epilogue = d->gated ? LEANFFN_EPI_GLU_FWD : LEANFFN_EPI_ACT_FWD;
      g.act = d->act;
      g.D2 = p.hid, g.ldd2 = I;
    }
    RUN(forward_product(d, &d->i2h, &g, p.xhat, H, N1, i2h_lowrank_hid, st));
    if (!fuse) RUN(leanffn_activation_forward(pre_activation, p.hid, LEANFFN_BF16, T, I, d->gated, d->act, st));
  }
  // output projection (+ low rank), bias + dropout + residual in its epilogue: ffn.py:191-207
  if (d->h2o.rank > 0)
    RUN(plain_product(d, p.hid, I, false, d->h2o.lowrank_first, I, false, T, d->h2o.rank, I, h2o_lowrank_hid, d->h2o.rank,
                      LEANFFN_BF16, st));
  {
    leanffn_gemm_desc g;
    base_desc(d, &g);
    g.epilogue = LEANFFN_EPI_DROPOUT_RESIDUAL;
    g.D = out, g.ldd = H;
    if (d->residual) g.aux = x, g.ldaux = H, g.aux_dtype = d->io_dtype;
    g.dropout_p = d->dropout_p, g.seed = d->seed, g.elem_offset = d->elem_offset;
    RUN(forward_product(d, &d->h2o, &g, p.hid, I, H, h2o_lowrank_hid, st));
  }
  return LEANFFN_OK;
}

extern "C" int32_t leanffn_ffn_backward(const leanffn_ffn_desc* d, const void* grad_out, const void* x,
                                        const void* pre_activation, const void* i2h_lowrank_hid,
                                        const void* h2o_lowrank_hid, const leanffn_ffn_grads* grads, void* workspace,
                                        void* stream) {
  NvtxRange range("leanffn_ffn_backward");
  RUN(validate(d));
  if (grads == nullptr) return LEANFFN_ERR_NULL;
  if ((grads->grad_ln_weight == nullptr) != (grads->grad_ln_bias == nullptr)) return LEANFFN_ERR_NULL;
  const int64_t T = d->tokens, H = d->hidden, I = d->intermediate, N1 = width1(d);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (T == 0) return LEANFFN_OK;  // nothing to add: the caller zero-fills gradients of an empty batch
  if (grad_out == nullptr || x == nullptr || pre_activation == nullptr || workspace == nullptr) return LEANFFN_ERR_NULL;
  if ((d->i2h.rank > 0 && i2h_lowrank_hid == nullptr) || (d->h2o.rank > 0 && h2o_lowrank_hid == nullptr)) return LEANFFN_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) % ALIGN != 0) return LEANFFN_ERR_ALIGN;
  const BwdPlan p = plan_backward(d, workspace);
  const int32_t wdt = d->param_dtype;  // weight-like gradients come back in the parameters' type

  // incoming gradient: mask of the forward (regenerated from seed / offset), cast, bias gradient of the output
  // projection: ffn.py:243-245, linear.py:293-294
  const void* dyp = grad_out;
  bool have_db2 = false;
  if (p.dyp != nullptr) {
    if (grads->grad_h2o_bias != nullptr) {
      RUN(leanffn_dropout_colsum(grad_out, d->grad_out_dtype, p.dyp, LEANFFN_BF16, T, H, d->dropout_p, d->seed,
                                 d->elem_offset, grads->grad_h2o_bias, p.scratch, st));
      have_db2 = true;
    } else {
      RUN(leanffn_dropout(grad_out, d->grad_out_dtype, p.dyp, LEANFFN_BF16, T * H, d->dropout_p, d->seed, d->elem_offset,
                          nullptr, 0, st));
    }
    dyp = p.dyp;
  }
  if (grads->grad_h2o_bias != nullptr && !have_db2)
    RUN(leanffn_column_sum(dyp, LEANFFN_BF16, H, grads->grad_h2o_bias, p.scratch, T, H, st));
  const void* dres = nullptr;
  if (d->residual) {
    dres = grad_out;
    if (p.dres != nullptr) {
      RUN(leanffn_cast(grad_out, d->grad_out_dtype, p.dres, LEANFFN_BF16, T * H, st));
      dres = p.dres;
    }
  }

  // output projection backward; its input-gradient epilogue applies the activation backward, rematerialises the
  // activation and emits the partial column sums of dPre: ffn.py:262-278
  if (d->h2o.rank > 0)
    RUN(plain_product(d, dyp, H, false, d->h2o.lowrank_second, d->h2o.rank, true, T, d->h2o.rank, H, p.glr2, d->h2o.rank,
                      LEANFFN_BF16, st));
  const bool want_db1 = grads->grad_i2h_bias != nullptr;
  {
    leanffn_gemm_desc g;
    base_desc(d, &g);
    g.epilogue = d->gated ? LEANFFN_EPI_GLU_BWD : LEANFFN_EPI_ACT_BWD;
    g.act = d->act;
    g.aux = pre_activation, g.ldaux = N1, g.aux_dtype = LEANFFN_BF16;
    g.D = p.dpre, g.ldd = N1;
    g.D2 = p.hid, g.ldd2 = I;
    if (want_db1) g.colsum_partial = p.partial, g.ld_colsum = N1;
    RUN(input_grad_product(d, &d->h2o, &g, dyp, I, H, p.glr2, st));
  }
  if (want_db1)
    RUN(leanffn_column_sum(p.partial, LEANFFN_F32, N1, grads->grad_i2h_bias, p.scratch, (T + 31) / 32, N1, st));
  if (grads->grad_h2o_weight != nullptr) RUN(weight_grad_product(d, &d->h2o, dyp, p.hid, I, H, grads->grad_h2o_weight, wdt, st));
  if (d->h2o.rank > 0 && grads->grad_h2o_lowrank_second != nullptr)
    RUN(plain_product(d, dyp, H, true, h2o_lowrank_hid, d->h2o.rank, true, H, d->h2o.rank, T, grads->grad_h2o_lowrank_second,
                      d->h2o.rank, wdt, st));
  if (d->h2o.rank > 0 && grads->grad_h2o_lowrank_first != nullptr)
    RUN(plain_product(d, p.glr2, d->h2o.rank, true, p.hid, I, true, d->h2o.rank, I, T, grads->grad_h2o_lowrank_first, I, wdt, st));

  // input projection backward on the rematerialised LayerNorm output: ffn.py:280-295, linear.py:296-328
  const bool need_xhat = grads->grad_i2h_weight != nullptr || (d->i2h.rank > 0 && grads->grad_i2h_lowrank_first != nullptr);
  if (need_xhat)
    RUN(leanffn_layer_norm_forward(x, d->io_dtype, d->ln_weight, d->ln_bias, d->param_dtype, p.xhat, LEANFFN_BF16, T, H,
                                   d->eps, 0.f, 0, 0, nullptr, 0, st));
  const bool need_input_side = grads->grad_input != nullptr || grads->grad_ln_weight != nullptr;
  if (d->i2h.rank > 0 && (need_input_side || grads->grad_i2h_lowrank_first != nullptr))
    RUN(plain_product(d, p.dpre, N1, false, d->i2h.lowrank_second, d->i2h.rank, true, T, d->i2h.rank, N1, p.glr1, d->i2h.rank,
                      LEANFFN_BF16, st));
  if (d->i2h.rank > 0 && grads->grad_i2h_lowrank_second != nullptr)
    RUN(plain_product(d, p.dpre, N1, true, i2h_lowrank_hid, d->i2h.rank, true, N1, d->i2h.rank, T,
                      grads->grad_i2h_lowrank_second, d->i2h.rank, wdt, st));
  if (d->i2h.rank > 0 && grads->grad_i2h_lowrank_first != nullptr)
    RUN(plain_product(d, p.glr1, d->i2h.rank, true, p.xhat, H, true, d->i2h.rank, H, T, grads->grad_i2h_lowrank_first, H, wdt, st));
  if (grads->grad_i2h_weight != nullptr) RUN(weight_grad_product(d, &d->i2h, p.dpre, p.xhat, H, N1, grads->grad_i2h_weight, wdt, st));
  if (need_input_side) {
    leanffn_gemm_desc g;
    base_desc(d, &g);
    g.D = p.dxhat, g.ldd = H;
    RUN(input_grad_product(d, &d->i2h, &g, p.dpre, H, N1, p.glr1, st));
    // LayerNorm backward + the residual's gradient: ffn.py:288-300
    RUN(leanffn_layer_norm_backward(p.dxhat, LEANFFN_BF16, x, d->io_dtype, d->ln_weight, d->param_dtype, dres, LEANFFN_BF16,
                                    grads->grad_input, d->io_dtype, grads->grad_ln_weight, grads->grad_ln_bias, p.scratch, T,
                                    H, d->eps, st));
  }
  return LEANFFN_OK;
}
