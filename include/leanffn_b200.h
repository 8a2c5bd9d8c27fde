/*
 * leanffn_b200.h -- C ABI of the B200 (sm_100a) LeanFFN / block-sparse linear kernels.
 *
 * Every entry point is `extern "C"`, takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), launches asynchronously on that stream and returns
 * an int32 status: 0 = ok, < 0 = rejected argument (nothing was launched), > 0 = CUDA runtime
 * error code + 1000.  No entry point allocates device memory (scratch is caller-provided)
 * unless its comment says otherwise; none synchronises the device.
 *
 * Device-side waits are bounded: a kernel that gives up on a wait records a non-zero word in
 * the caller-provided `status_word` (int32 in device memory, may be NULL) and returns.
 *
 * The entry points replace, one to one, what the reference (learning-at-home/lean_transformer)
 * asks of PyTorch/ATen/cuBLAS/Triton on its LeanFFN path.  Each declaration cites the reference
 * call site it stands in for (file:line relative to the reference project root).
 */
#ifndef LEANFFN_B200_H_
#define LEANFFN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums (plain ints in the ABI) ------------------------------------------------------ */

/* element types */
#define LEANFFN_F32 0
#define LEANFFN_BF16 1
#define LEANFFN_TF32 2 /* leanffn_gemm in_dtype only: fp32 storage, TF32 multiplication on the tensor cores */

/* activations: lean_transformer/utils.py:24-38 (gelu_fused) and the transformers ACT2FN names
 * the reference re-exports at lean_transformer/utils.py:80 */
#define LEANFFN_ACT_GELU_TANH 0 /* gelu_fused, gelu_new, gelu_pytorch_tanh: 0.5x(1+tanh(0.79788456 x (1+0.044715 x^2))) */
#define LEANFFN_ACT_GELU_ERF 1  /* gelu */
#define LEANFFN_ACT_RELU 2
#define LEANFFN_ACT_SILU 3      /* silu, swish */
#define LEANFFN_ACT_TANH 4
#define LEANFFN_ACT_SIGMOID 5
#define LEANFFN_ACT_IDENTITY 6  /* linear */
#define LEANFFN_ACT_COUNT 7

/* GEMM epilogues */
#define LEANFFN_EPI_STORE 0            /* D = acc [+ bias] */
#define LEANFFN_EPI_GLU_FWD 1          /* gated: D = pre (acc+bias, [M,2I]), D2 = act(pre[:, :I]) * pre[:, I:] */
#define LEANFFN_EPI_ACT_FWD 2          /* D = pre (acc+bias), D2 = act(pre) */
#define LEANFFN_EPI_DROPOUT_RESIDUAL 3 /* D = dropout(acc+bias) + aux */
#define LEANFFN_EPI_GLU_BWD 4          /* acc = dHid [M,I]; aux = pre [M,2I]; D = dPre [M,2I]; D2 = hid (optional) */
#define LEANFFN_EPI_ACT_BWD 5          /* acc = dHid [M,N]; aux = pre; D = acc * act'(pre); D2 = act(pre) (optional) */

/* negative status codes */
#define LEANFFN_OK 0
#define LEANFFN_ERR_NULL (-1)
#define LEANFFN_ERR_SHAPE (-2)
#define LEANFFN_ERR_ALIGN (-3)
#define LEANFFN_ERR_DTYPE (-4)
#define LEANFFN_ERR_UNSUPPORTED (-5)
#define LEANFFN_ERR_DRIVER (-6)   /* could not obtain / call cuTensorMapEncodeTiled */
#define LEANFFN_ERR_TOO_LARGE (-7)

/* device-side status_word values */
#define LEANFFN_DEV_OK 0
#define LEANFFN_DEV_TIMEOUT_PRODUCER 1
#define LEANFFN_DEV_TIMEOUT_MMA 2
#define LEANFFN_DEV_TIMEOUT_EPILOGUE 3
#define LEANFFN_DEV_TIMEOUT_PEER 4 /* leanffn_peer_barrier: a rank did not arrive within the limit */

/* Version of this header; leanffn_abi_version() returns the one the library was built from. */
#define LEANFFN_ABI_VERSION 4
int32_t leanffn_abi_version(void);
const char* leanffn_status_string(int32_t status);

/* ---- row kernels ------------------------------------------------------------------------ */

/* LayerNorm forward over the last dim: y = (x - mean) * rsqrt(var + eps) * gamma + beta, biased
 * variance, statistics in fp32 (two-pass over registers).  Optionally followed by
 * y = dropout(y) (Philox mask, see leanffn_dropout) and y += residual.
 * Replaces F.layer_norm at lean_transformer/ffn.py:184, :200 and :283, torch.dropout_ at :204
 * and torch.add at :207 (post-LN configuration). x, residual: x_dtype; gamma, beta: param_dtype
 * (may be NULL = ones / zeros); y: y_dtype.  Pointers that are not 16-byte aligned (or cols % 4 != 0) take a
 * slower scalar kernel. */
int32_t leanffn_layer_norm_forward(const void* x, int32_t x_dtype, const void* gamma, const void* beta,
                                   int32_t param_dtype, void* y, int32_t y_dtype, int64_t rows, int64_t cols,
                                   float eps, float dropout_p, uint64_t seed, uint64_t elem_offset,
                                   const void* residual, int32_t residual_dtype, void* stream);

/* Scratch (bytes) leanffn_layer_norm_backward needs for its per-block partial sums. */
size_t leanffn_layer_norm_backward_scratch_bytes(int64_t rows, int64_t cols);

/* LayerNorm backward with statistics recomputed from x (nothing but x is read from the forward):
 *   dx = rstd * (g - mean(g) - xn * mean(g * xn)) [+ dresidual],  g = dy * gamma,
 *   dgamma = sum_rows(dy * xn), dbeta = sum_rows(dy).
 * Replaces torch.autograd.grad over the rematerialised F.layer_norm at
 * lean_transformer/ffn.py:247-259 and :280-293, and the residual add at :297-300.
 * dgamma/dbeta are fp32 [cols] (may be NULL together); dx may be NULL.  With cols % 4 == 0 and cols <= 16384 every
 * pointer must be 16-byte aligned (LEANFFN_ERR_ALIGN otherwise). */
int32_t leanffn_layer_norm_backward(const void* dy, int32_t dy_dtype, const void* x, int32_t x_dtype,
                                    const void* gamma, int32_t param_dtype, const void* dresidual,
                                    int32_t dresidual_dtype, void* dx, int32_t dx_dtype, float* dgamma,
                                    float* dbeta, void* scratch, int64_t rows, int64_t cols, float eps,
                                    void* stream);

/* hid = act(pre) (gated == 0, pre [rows, inter]) or act(pre[:, :inter]) * pre[:, inter:]
 * (gated != 0, pre [rows, 2*inter]).  Replaces _LeanFFN._apply_activation,
 * lean_transformer/ffn.py:138-144 (the first half of the last dim is the gate).  inter % 4 == 0 and 16-byte
 * aligned pointers are required (LEANFFN_ERR_SHAPE / LEANFFN_ERR_ALIGN); the same holds for the backward. */
int32_t leanffn_activation_forward(const void* pre, void* hid, int32_t dtype, int64_t rows, int64_t inter,
                                   int32_t gated, int32_t act, void* stream);

/* dpre = d(hid)/d(pre) applied to dhid; optionally also rematerialises hid (hid_out may be NULL).
 * Replaces torch.autograd.grad(hid_act, pre_activation, ...) at lean_transformer/ffn.py:275
 * (GELU.backward, lean_transformer/utils.py:33-50). */
int32_t leanffn_activation_backward(const void* dhid, const void* pre, void* dpre, void* hid_out,
                                    int32_t dtype, int64_t rows, int64_t inter, int32_t gated, int32_t act,
                                    void* stream);

/* y[i] = (keep(seed, elem_offset + i) ? x[i] / (1 - p) : 0) [+ residual[i]], i in [0, n); residual may be
 * NULL.  keep() is a pure function:
 * Philox4x32-10 with key (seed_lo, seed_hi), counter ((e >> 2) lo, (e >> 2) hi, 0, 0), word e & 3,
 * keep iff word >= floor(p * 2^32).  The same call with the same (seed, offset) regenerates the
 * mask, which is how backward reuses the forward's mask.
 * Replaces torch.dropout_/torch.dropout at lean_transformer/ffn.py:204 and :245 (the reference
 * restores the RNG state instead, :308-321) and torch.add at :207. */
int32_t leanffn_dropout(const void* x, int32_t x_dtype, void* y, int32_t y_dtype, int64_t n, float p,
                        uint64_t seed, uint64_t elem_offset, const void* residual, int32_t residual_dtype,
                        void* stream);

/* y = dropout(x) cast to y_dtype over a [rows, cols] matrix (contiguous), and colsum[c] = sum_r y[r, c] of the rounded
 * values, in one pass over x: the first step of the backward, where the incoming gradient is masked with the
 * forward's mask, cast to the compute type and summed into the output projection's bias gradient.
 * Replaces torch.dropout at lean_transformer/ffn.py:245 followed by grad_output.sum(0) at
 * lean_transformer/blocksparse/linear.py:293-294.  p == 0 makes it a cast + column sum.  scratch: at least
 * leanffn_dropout_colsum_scratch_bytes(rows, cols) bytes, 16-byte aligned. */
size_t leanffn_dropout_colsum_scratch_bytes(int64_t rows, int64_t cols);
int32_t leanffn_dropout_colsum(const void* x, int32_t x_dtype, void* y, int32_t y_dtype, int64_t rows, int64_t cols,
                               float p, uint64_t seed, uint64_t elem_offset, float* colsum, void* scratch,
                               void* stream);

/* mask[i] = keep(seed, elem_offset + i) as uint8; lets a checker inject the very same mask into
 * another implementation. */
int32_t leanffn_dropout_mask(uint8_t* mask, int64_t n, float p, uint64_t seed, uint64_t elem_offset,
                             void* stream);

size_t leanffn_column_sum_scratch_bytes(int64_t rows, int64_t cols);
/* out[c] = sum_r x[r, c] in fp32, deterministic two-stage reduction.  x may be any view with ld >= cols; rows
 * are read with 4-element vector loads when the base address and ld allow it, element by element otherwise.
 * Replaces grad_output_flat.sum(dim=0) at lean_transformer/blocksparse/linear.py:293-294. */
int32_t leanffn_column_sum(const void* x, int32_t x_dtype, int64_t ld, float* out, void* scratch,
                           int64_t rows, int64_t cols, void* stream);

/* Same result as leanffn_column_sum, for callers that cannot hand over scratch memory: a host that drives
 * this library through the C ABI alone has no tensor allocator behind it, and a serving or training process
 * that has given the whole device to its own pool (or that must not stall on the implicit synchronisation of
 * cudaMalloc / cudaFree in its steady state) cannot allocate at call time.  The partial sums go to a fixed
 * 1 MiB array inside the library image instead; every GPU that loads the library holds that array until the
 * process exits.  The call allocates and frees nothing.
 * Limit: any number of rows, at most 65536 columns (wider inputs, or a GPU so large that its partial sums
 * exceed leanffn_column_sum_static_capacity() = 262144 floats, are rejected with LEANFFN_ERR_TOO_LARGE and
 * nothing is launched).
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call outside any stream capture.  All calls on a device share the one array:
 * calls that may overlap on the GPU (different streams without ordering) race on it and must be serialised
 * by the caller.  The array keeps whatever the last call left; each call overwrites every partial it reads,
 * so no clearing is needed.
 * No counterpart in the reference: it has no C ABI and allocates through PyTorch everywhere. */
int64_t leanffn_column_sum_static_capacity(void);
int32_t leanffn_column_sum_static(const void* x, int32_t x_dtype, int64_t ld, float* out, int64_t rows,
                                  int64_t cols, void* stream);

/* y = (y_dtype) x, n elements. Replaces the autocast casts the reference relies on
 * (torch.cuda.amp.custom_fwd at lean_transformer/ffn.py:147). */
int32_t leanffn_cast(const void* x, int32_t x_dtype, void* y, int32_t y_dtype, int64_t n, void* stream);

/* y[c, r] = x[r, c]; x is [rows, cols] with leading dim ldx, y is [cols, rows] contiguous. */
int32_t leanffn_transpose(const void* x, int32_t dtype, int64_t ldx, void* y, int64_t rows, int64_t cols,
                          void* stream);

/* ---- GEMMs ------------------------------------------------------------------------------ */

/* One descriptor serves the dense and the block-sparse products and all fused epilogues.
 *
 * D[M,N] = sum over k of A(m,k) * B(n,k), fp32 accumulation.
 *   a_mn_major == 0: A is stored [M,K] row-major (K contiguous, leading dim lda)
 *   a_mn_major != 0: A is stored [K,M] row-major (M contiguous)            -- "transposed"
 *   b_mn_major == 0: B is stored [N,K] row-major (K contiguous)            -- x @ W^T with W [out,in]
 *   b_mn_major != 0: B is stored [K,N] row-major (N contiguous)
 * This covers lean_transformer/blocksparse/linear.py:219 (F.linear), :304-305 (wgrad, both
 * operands MN-major, K = tokens) and :307-308 (dgrad, B MN-major).
 *
 * Low-rank term (optional, lean_transformer/blocksparse/linear.py:221-226 and :317-323): after the
 * main k-loop the kernel continues over a second operand pair A2 (M x K2) / B2 (N x K2), stored with
 * the same majorness as A / B, accumulating into the same tile.
 *
 * Block-sparse modes (lean_transformer/blocksparse/native_backend.py:9-76 and the Triton operator of
 * lean_transformer/blocksparse/triton_backend.py:18-79).  B is an array of bs_num_blocks weight blocks,
 * block f a row-major [block(out) x block(in)] matrix at B + f*block*block.  That is the reference's
 * native tensor [in_features, blocks_per_input, block] (f = j*blocks_per_input + a) as well as its
 * Triton tensor [1, nnz, block, block] (f = rank of the block in layout.nonzero()).  Which blocks meet
 * is given by bs_index, a table of int32 PAIRS with bs_nnz pairs per row, and bs_count (int32 per
 * table row: how many leading pairs are valid; NULL = bs_nnz everywhere):
 * Table entries are TRUSTED: the kernels use them as block addresses without range checks, so the caller
 * validates tables that come from outside (lean_transformer_b200 does so when it first builds them).
 *   bs_mode 0: dense.
 *   bs_mode 1: forward.  A = x [M, K=in_features], N = out_features.  Table row = output block,
 *              pair = (weight block f, input block j):  D[:, i] = sum_t x[:, j_t] . W_f_t^T.
 *   bs_mode 2: dgrad.    A = dy [M, K=out_features], N = in_features.  Table row = input block,
 *              pair = (weight block f, output block o): D[:, j] = sum_t dy[:, o_t] . W_f_t.
 *   bs_mode 3: wgrad.    A = dy [tokens(K), out_features] and B = x [tokens(K), in_features], both
 *              MN-major; D = the weight gradient, M = bs_num_blocks*block rows of N = block columns.
 *              Table row = weight block f, one pair (output block o, input block j), bs_nnz = 1.
 * Block-sparse products take LEANFFN_EPI_STORE; the input-gradient mode (2) also takes LEANFFN_EPI_GLU_BWD and
 * LEANFFN_EPI_ACT_BWD (the epilogue reads the dense pre-activation tensor, which the sparsity does not touch); the
 * forward mode (1) also takes LEANFFN_EPI_DROPOUT_RESIDUAL and, for bf16 with bs_block == 128 and N/2 a multiple
 * of 128, LEANFFN_EPI_GLU_FWD.  For the latter the CALLER guarantees that table rows i and i + N/(2*bs_block)
 * (a gate block and its linear partner) list the same input blocks in the same order and have equal bs_count:
 * one activation tile then meets the weight blocks of both halves (true for pixelfly layouts, whose pattern
 * repeats along the output dimension).
 */
typedef struct leanffn_gemm_desc {
  int32_t M, N, K;
  int32_t in_dtype;      /* LEANFFN_BF16: tcgen05 tensor-core path; LEANFFN_F32: SIMT fp32 path;
                            LEANFFN_TF32: fp32 operands on the tensor cores, see leanffn_split_tf32 */
  const void* A;
  int64_t lda;
  int32_t a_mn_major;
  int32_t b_mn_major;
  const void* B;
  int64_t ldb;
  /* low-rank continuation (K2 == 0 disables) */
  const void* A2;
  const void* B2;
  int64_t lda2, ldb2;
  int32_t K2;
  /* block-sparse */
  int32_t bs_mode;
  int32_t bs_block;
  int32_t bs_nnz;        /* pairs per row of bs_index */
  int32_t bs_num_blocks; /* number of weight blocks in B (modes 1, 2) or D (mode 3) */
  const int32_t* bs_index;
  const int32_t* bs_count;
  /* epilogue */
  int32_t epilogue;
  int32_t act;
  void* D;
  int64_t ldd;
  int32_t d_dtype;
  void* D2;
  int64_t ldd2;
  const void* bias;  /* [N] or NULL */
  int32_t bias_dtype;
  const void* aux;   /* residual [M,N] or pre-activation, see epilogue */
  int64_t ldaux;
  int32_t aux_dtype;
  float dropout_p;
  uint64_t seed;
  uint64_t elem_offset; /* element index of D[0,0] in the logical dropout stream */
  int32_t* status_word; /* device int32 or NULL */
  int32_t force_simt;   /* != 0: run the SIMT kernel whatever the dtype (checker / odd shapes) */
  int32_t max_ctas;     /* > 0: cap on the persistent grid of the tensor-core kernel (leave SMs to a
                           concurrently running collective); 0 = one CTA per SM */
  /* Reduce-scatter fused into the epilogue (data-parallel weight gradients; no counterpart in the reference, which
   * has no distributed code).  scatter_world = W > 0 (at most 8): the result is not stored to D; element (r, c) is
   * ADDED (relaxed atomic add at system scope) to scatter_D[(r >> scatter_block_shift) % W] + r*ldd + c, where
   * scatter_D[k] is the address of the SAME [M, ldd] matrix in the memory of rank k (peer-mapped over NVLink; entry
   * [own rank] is local).  After every rank has run its product and the ranks have synchronised, rank k holds the
   * sum over ranks of the row blocks it owns (blocks of 2^scatter_block_shift rows, dealt round-robin); the other
   * rows of its replica are untouched.  The caller zeroes the owned blocks before the first contribution can
   * arrive.  Tensor-core path with LEANFFN_EPI_STORE, no bias, scatter_block_shift >= 7 only. */
  int32_t scatter_world;
  int32_t scatter_block_shift;
  void* scatter_D[8];
  /* bs_mode 3 with bs_block == 128 only: != 0 asserts that weight blocks 2i and 2i+1 read the same input block
   * (equal second entries of their table rows; bs_num_blocks even), as in the reference's native order with an
   * even number of blocks per input block.  One CTA then computes both blocks from one tile of x. */
  int32_t bs_wgrad_pairs;
  /* SM clocks a warp role of the tensor-core kernel waits on a stalled peer role before it gives up and records a
   * LEANFFN_DEV_TIMEOUT_* code in status_word (0 = the default, about 2e9 clocks = one second). */
  int64_t wait_limit_cycles;
  /* LEANFFN_EPI_GLU_BWD / LEANFFN_EPI_ACT_BWD only (may be NULL): the bias gradient of the layer in front of the
   * activation, db = D.sum(rows) (lean_transformer/blocksparse/linear.py:293-294), rides in this epilogue.  The
   * kernel writes fp32 partial sums, one row per 32 rows of D: colsum_partial[(r / 32) * ld_colsum + c] = sum of the
   * stored (rounded) D[r', c] over the rows r' of that group; ceil(M / 32) rows of as many columns as D has.
   * leanffn_column_sum over those partial rows finishes the reduction (deterministic). */
  float* colsum_partial;
  int64_t ld_colsum;
  /* Optional (NULL = off): a timer made by leanffn_timer_create.  The call then records a CUDA event pair around its
   * kernel on `stream` and books the launch's algorithmic FLOPs (2 * M * N * (K_effective + K2)) with it. */
  void* timer;
  /* in_dtype LEANFFN_TF32 only: > 0 cuts the reduction axis into slices of this many elements (a multiple of 96: three
   * parts of a multiple of 32), the last slice taking the remainder, i.e. the slices leanffn_split_tf32 lays out for
   * slice width tf32_k_slice / 3.  The kernel accumulates every slice in tensor memory on its own and keeps the
   * running fp32 sum in D, so one launch gives what one launch per slice (with aux = D) would. */
  int32_t tf32_k_slice;
} leanffn_gemm_desc;

int32_t leanffn_gemm(const leanffn_gemm_desc* desc, void* stream);

/* ---- timing of GEMM launches ---------------------------------------------------------------------- */

/* A timer owns `capacity` CUDA event pairs (created here, once: nothing is allocated while it is in use).  Every
 * leanffn_gemm call whose descriptor names the timer (directly, or through leanffn_ffn_desc.timer) records one pair
 * around its kernel on the launching stream and notes the launch's algorithmic FLOPs; launches beyond the capacity
 * are counted but not timed.  leanffn_timer_summary synchronises on the recorded events and returns the sums over the
 * timed launches; leanffn_timer_reset forgets them.  One timer serves one device and one host thread at a time.
 * No counterpart in the reference (it times with torch.profiler from outside). */
int32_t leanffn_timer_create(int32_t capacity, void** timer);
int32_t leanffn_timer_reset(void* timer);
int32_t leanffn_timer_summary(void* timer, double* flops, double* seconds, int32_t* timed_launches,
                              int32_t* dropped_launches);
int32_t leanffn_timer_destroy(void* timer);

/* ---- the whole block in one call ---------------------------------------------------------------------- */

/* One projection of the block (lean_transformer/blocksparse/linear.py:19-149): a dense [out, in] weight, or an
 * array of bs_block x bs_block weight blocks with the three pair tables of leanffn_gemm (forward / dgrad / wgrad;
 * see bs_mode above), plus an optional low-rank pair and bias.  Weights and low-rank factors are given in the
 * compute type (bf16); masters kept in fp32 are converted by the caller. */
typedef struct leanffn_linear_desc {
  const void* weight;
  const void* bias; /* [out] or NULL */
  int32_t bias_dtype;
  int32_t rank;               /* 0: no low-rank term; else a multiple of 8 */
  const void* lowrank_first;  /* [rank, in]  */
  const void* lowrank_second; /* [out, rank] */
  int32_t bs_block;           /* 0: dense */
  int32_t bs_num_blocks;
  const int32_t* fwd_index;
  const int32_t* fwd_count; /* may be NULL */
  int32_t fwd_nnz;
  int32_t dgrad_nnz;
  const int32_t* dgrad_index;
  const int32_t* dgrad_count; /* may be NULL */
  const int32_t* wgrad_index;
  int32_t wgrad_pairs;        /* see leanffn_gemm_desc.bs_wgrad_pairs */
  int32_t fuse_gated_forward; /* block-sparse input projection of a gated block: the caller guarantees what
                                 LEANFFN_EPI_GLU_FWD asks of the forward table (gate / linear rows pair up) */
} leanffn_linear_desc;

/* The block: lean_transformer/ffn.py:35-64 (module) and :148-175 (the autograd function's arguments).
 * Compute type bf16 (fp32 accumulation); the residual stream x / grad_input is io_dtype (fp32 or bf16); LayerNorm
 * parameters and all parameter gradients are param_dtype (fp32 masters under autocast, or bf16), bias gradients and
 * LayerNorm gradients always fp32.  Without the post-LayerNorm option (post_layer_norm=True is driven piecewise). */
typedef struct leanffn_ffn_desc {
  int64_t tokens;
  int32_t hidden, intermediate;
  int32_t gated, act, residual;
  int32_t compute_dtype;  /* LEANFFN_BF16 */
  int32_t io_dtype;       /* x, grad_input */
  int32_t grad_out_dtype; /* the gradient arriving at the block's output */
  int32_t param_dtype;    /* ln_weight / ln_bias, weight-like gradients */
  float eps;
  float dropout_p;        /* 0: no dropout (evaluation, or p = 0) */
  uint64_t seed, elem_offset;
  const void* ln_weight; /* may be NULL (ones) */
  const void* ln_bias;   /* may be NULL (zeros) */
  leanffn_linear_desc i2h, h2o;
  int32_t* status_word; /* see leanffn_gemm_desc */
  int32_t max_ctas;
  void* timer;          /* see leanffn_gemm_desc */
} leanffn_ffn_desc;

/* Where the backward puts each gradient; NULL = not needed (the work is skipped where that is possible).
 * Weight-like gradients have the weight's own shape and storage order in param_dtype; bias and LayerNorm
 * gradients are fp32 vectors (grad_ln_weight and grad_ln_bias come together or not at all). */
typedef struct leanffn_ffn_grads {
  void* grad_input;
  float* grad_ln_weight;
  float* grad_ln_bias;
  void* grad_i2h_weight;
  float* grad_i2h_bias;
  void* grad_i2h_lowrank_first;
  void* grad_i2h_lowrank_second;
  void* grad_h2o_weight;
  float* grad_h2o_bias;
  void* grad_h2o_lowrank_first;
  void* grad_h2o_lowrank_second;
} leanffn_ffn_grads;

/* Bytes of workspace leanffn_ffn_forward (backward == 0) or leanffn_ffn_backward (backward != 0) needs for this
 * descriptor; 0 for a descriptor the calls would reject.  The workspace must be 256-byte aligned. */
size_t leanffn_ffn_workspace_bytes(const leanffn_ffn_desc* desc, int32_t backward);

/* out = [x +] dropout(act(LN(x) . W1^T + b1) . W2^T + b2), the forward of lean_transformer/ffn.py:146-217.
 * x [tokens, hidden] io_dtype; out [tokens, hidden] bf16; pre_activation [tokens, intermediate * (1 + gated)] bf16 is
 * written for the backward (with x it is all the backward needs: ffn.py:209-216), as are the low-rank hidden states
 * [tokens, rank] bf16 of projections that have a low-rank term (NULL otherwise). */
int32_t leanffn_ffn_forward(const leanffn_ffn_desc* desc, const void* x, void* out, void* pre_activation,
                            void* i2h_lowrank_hid, void* h2o_lowrank_hid, void* workspace, void* stream);

/* The memory-lean backward of lean_transformer/ffn.py:220-306: the dropout mask is regenerated from (seed,
 * elem_offset), the activation and the LayerNorm output are rematerialised from pre_activation and x. */
int32_t leanffn_ffn_backward(const leanffn_ffn_desc* desc, const void* grad_out, const void* x,
                             const void* pre_activation, const void* i2h_lowrank_hid, const void* h2o_lowrank_hid,
                             const leanffn_ffn_grads* grads, void* workspace, void* stream);

/* Self-test of the bounded device-side wait: launches one warp whose thread 0 waits, for at most limit_cycles SM
 * clocks (clamped to [1000, 10000000]), on an mbarrier that nothing ever arrives at.  The wait gives up, the kernel
 * records LEANFFN_DEV_TIMEOUT_EPILOGUE in *status_word with the same code path the GEMM roles use, and returns;
 * nothing hangs or traps and the context stays usable.  Lets a host-side test exercise "a wait ran out -> status
 * word -> error on the host" without stalling a real kernel.  No counterpart in the reference. */
int32_t leanffn_selftest_wait_timeout(int32_t* status_word, int64_t limit_cycles, void* stream);

/* fp32 accuracy from TF32 tensor-core multiplications ("3xTF32").  A TF32 multiplication reads only the 10 leading
 * mantissa bits of each fp32 operand.  Write x = hi + lo with hi = x truncated to those bits and lo = x - hi; then
 * a.b = a_hi.b_hi + a_hi.b_lo + a_lo.b_hi up to a relative 2^-21, and the three products are ONE product over a
 * reduction axis of three times the length.  Tensor-core accumulators truncate, so the error of such a product grows
 * with the length of its reduction axis; a long axis is therefore cut into slices that are multiplied by separate
 * calls keeping a running sum.  This call prepares all slices at once.  For x [rows, cols] (leading dimension ldx)
 * and a slice width s, the columns are cut into max(1, cols / s) slices (the last one takes the remainder), and
 * slice j, covering columns [f, f + w), lands in out [rows, 3*cols] at columns [3f, 3f + 3w) as
 *   role 0 (the A operand):  ( hi | lo | hi )        role 1 (the B operand):  ( lo | hi | hi ),   each part w wide
 * (the two small cross products come first, so that they add up before the accumulator has grown and only the
 * last third of the slice truncates an accumulator of full size).
 * leanffn_gemm with in_dtype LEANFFN_TF32, A = outA + 3f, B = outB + 3f, lda = ldb = 3*cols and K = 3w then
 * gives the fp32-accurate product over that slice (K-major operands, dense, LEANFFN_EPI_STORE with optional bias,
 * fp32 result, M, N >= 64, N a multiple of 8, f and w multiples of 4).  With in_dtype LEANFFN_TF32, `aux`
 * (fp32 [M, N], may be D itself) is added to the result: that is the running sum over slices.  ONE call covers all
 * slices when the descriptor's tf32_k_slice = 3w is set (A = outA, B = outB, K = 3*cols; w a multiple of 32).
 * Stands in for the fp32 cuBLAS products of the reference's fp32 (non-autocast) mode. */
int32_t leanffn_split_tf32(const float* x, int64_t ldx, float* out, int64_t rows, int64_t cols, int32_t role,
                           int64_t slice, void* stream);

/* Barrier between the ranks of one NVLink domain (at most 8 GPUs, one process per GPU) with a BOUNDED wait and no
 * trap: rank r stores `epoch` into slot [channel][r] of every peer's flag array (release, system scope) and waits
 * until every slot [channel][t] of its own array holds a value >= epoch (acquire loads).  flags[t] is the address,
 * valid on this GPU, of rank t's flag array: 4 channels x 8 uint32, zero-initialised once, peer-mapped (for example
 * a region of a symmetric-memory buffer).  Every rank calls with the same (channel, epoch); epochs of a channel
 * increase by one per barrier (wrap-around safe).  A rank that waits longer than limit_cycles SM clocks (0 = about
 * 20 s) records LEANFFN_DEV_TIMEOUT_PEER in *status_word and returns: nothing hangs, the host reads the word and
 * decides.  Writes made by earlier kernels of this stream are visible to the peers' kernels that follow their
 * barrier.  One warp, no shared memory: it fits beside a persistent GEMM that leaves one SM free.
 * No counterpart in the reference (it has no distributed code). */
int32_t leanffn_peer_barrier(void* const* flags, int32_t rank, int32_t world, int32_t channel, uint32_t epoch,
                             int64_t limit_cycles, int32_t* status_word, void* stream);

/* Strided device-to-device copy of `height` pieces of `width_bytes` (cudaMemcpy2DAsync; between two GPUs with peer
 * access it runs on a copy engine and occupies no SM).  Used to hand the reduced row blocks of a scattered weight
 * gradient to the other ranks.  No counterpart in the reference. */
int32_t leanffn_copy_2d(void* dst, uint64_t dst_pitch_bytes, const void* src, uint64_t src_pitch_bytes,
                        uint64_t width_bytes, uint64_t height, void* stream);

/* ---- attention core -------------------------------------------------------------------------- */

/* Scaled dot-product attention over heads without materialising the [q_len, kv_len] matrices:
 *   out[b, q, h, :] = softmax_k(scale * <Q[b, q, h, :], K[b, k, h, :]> + mask[b, h, q, k]) . V[b, k, h, :]
 * Replaces SimpleAttentionCore._attention_core_forward (lean_transformer/attn.py:111-149: the key scaling at :125-126,
 * both torch.matmul calls at :132 and :146, the mask addition at :135, torch.softmax at :138, the head transposes at
 * :117-129 and :147) and what autograd derives from it in the backward pass.
 *
 * q, k, v, out, d_out, dk, dv are bf16 [batch, len, heads * head_dim] with a row pitch ld_* (elements), so the three
 * slices of one fused qkv projection output can be passed in place (attn.py:56-57).  head_dim is a multiple of 16,
 * at most 128; pointers 16-byte aligned, pitches multiples of 8.
 * mask: optional fp32 additive mask addressed as mask[b * mask_stride_b + h * mask_stride_h + q * mask_stride_q + k]
 * (stride 0 broadcasts; 0 where attention is allowed, a large negative number where it is not, attn.py:99).
 * causal != 0 additionally forbids k > q + (kv_len - q_len) and skips the tiles that rule empties.
 * lse: fp32 [batch, heads, q_len], log2 of the softmax denominator with the row maximum folded in, written by the
 * forward call and read by the backward call.
 * dropout_p > 0: dropout on the attention probabilities (attn.py:141-144): probability (b, h, q, k) is kept iff the
 * Philox word of element index elem_offset + ((b * heads + h) * q_len + q) * kv_len + k passes the threshold (the
 * mask function of leanffn_dropout), kept ones are scaled by 1 / (1 - p); forward and backward must be given the same
 * (dropout_p, seed, elem_offset).
 *
 * Backward needs, besides the forward's q, k, v, out and lse: delta (fp32 [batch, heads, q_len], scratch),
 * dq_accum (fp32 [batch, q_len, heads * head_dim] contiguous, zeroed by the call, receives dQ; convert / un-rotate it
 * with leanffn_rotary), dk and dv (bf16).  Device waits are bounded (status_word, wait_limit_cycles as in
 * leanffn_gemm_desc). */
typedef struct leanffn_attention_desc {
  int32_t batch, heads, q_len, kv_len, head_dim;
  int32_t causal;
  float scale;
  float dropout_p;
  const void* q;
  const void* k;
  const void* v;
  int64_t ld_q, ld_k, ld_v;
  const float* mask;
  int64_t mask_stride_b, mask_stride_h, mask_stride_q;
  void* out;
  int64_t ld_out;
  float* lse;
  /* backward only */
  const void* d_out;
  int64_t ld_dout;
  float* delta;
  float* dq_accum;
  void* dk;
  void* dv;
  int64_t ld_dk, ld_dv;
  int32_t* status_word;
  int64_t wait_limit_cycles;
  uint64_t seed;
  uint64_t elem_offset;
} leanffn_attention_desc;

int32_t leanffn_attention_forward(const leanffn_attention_desc* desc, void* stream);
int32_t leanffn_attention_backward(const leanffn_attention_desc* desc, void* stream);

/* Rotary position embedding over [batch, len, heads, head_dim] (lean_transformer/rotary.py:63-68, applied to queries
 * and keys at attn.py:163-171):  y = x * cos + rotate_half(x) * sin with rotate_half(x) = (-x_right, x_left) and
 * cos / sin fp32 tables [>= len, head_dim] (row pitch ld_table) as rotary.py:48-60 builds them; arithmetic in fp32,
 * one rounding to y_dtype.  inverse != 0 applies the transposed rotation (the backward pass: y = x * cos -
 * rotate_half(x * sin)).  cos == NULL copies / converts without rotating.  x: row pitch ld_x, y: row pitch ld_y
 * (elements); head_dim even. */
int32_t leanffn_rotary(const void* x, int32_t x_dtype, int64_t ld_x, const float* cos_table, const float* sin_table,
                       int64_t ld_table, void* y, int32_t y_dtype, int64_t ld_y, int32_t batch, int32_t len,
                       int32_t heads, int32_t head_dim, int32_t inverse, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LEANFFN_B200_H_ */
