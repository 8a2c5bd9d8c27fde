// Pieces shared by the SIMT and the tcgen05 GEMM kernels: the epilogue parameter block and the
// per-element / per-run epilogue math (bias, gated activation forward and backward, dropout,
// residual).
#pragma once
#include "math.cuh"

namespace leanffn {

struct EpiParams {
  int32_t kind;  // LEANFFN_EPI_*
  int32_t act;
  int32_t M, N;  // logical extent of the accumulator matrix
  void* D;
  int64_t ldd;
  int32_t d_dtype;
  void* D2;
  int64_t ldd2;
  const void* bias;
  int32_t bias_dtype;
  const void* aux;
  int64_t ldaux;
  int32_t aux_dtype;
  uint32_t threshold;  // 0: no dropout
  float keep_scale;
  uint64_t seed;
  uint64_t elem_offset;
  // reduce-scatter of the result into peer replicas (scatter_world == 0: plain store to D)
  int32_t scatter_world;
  int32_t scatter_shift;
  void* scatter_D[8];
  // activation-backward kinds: per-32-row partial column sums of D (the bias gradient), fp32 [ceil(M/32), ldcolsum]
  float* colsum;
  int64_t ldcolsum;
  int32_t ablate;  // measurement builds only (LEANFFN_ABLATE_RUNTIME): bit mask of epilogue phases to leave out
};

__device__ __forceinline__ float load_any(const void* p, int32_t dtype, int64_t i) {
  return dtype == LEANFFN_BF16 ? __bfloat162float(static_cast<const bf16*>(p)[i]) : static_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_any(void* p, int32_t dtype, int64_t i, float v) {
  if (dtype == LEANFFN_BF16)
    static_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
  else
    static_cast<float*>(p)[i] = v;
}

// Scalar epilogue for the kinds the SIMT kernel fuses (STORE, DROPOUT_RESIDUAL).
__device__ __forceinline__ void epilogue_scalar(const EpiParams& p, int64_t row, int64_t col, float acc) {
  if (p.bias != nullptr) acc += load_any(p.bias, p.bias_dtype, col);
  if (p.kind == LEANFFN_EPI_DROPOUT_RESIDUAL) {
    if (p.threshold != 0u)
      acc = dropout_keep1(p.elem_offset + static_cast<uint64_t>(row) * p.N + col, p.seed, p.threshold)
                ? acc * p.keep_scale
                : 0.f;
    if (p.aux != nullptr) acc += load_any(p.aux, p.aux_dtype, row * p.ldaux + col);
  }
  store_any(p.D, p.d_dtype, row * p.ldd + col, acc);
}

// ---- operand / parameter blocks shared between the entry point and the kernels ------------------
struct SimtOperands {
  const void* A;
  const void* B;
  int64_t a_sm, a_sk;  // element strides of A over (m, k)
  int64_t b_sn, b_sk;
  int32_t K;
  // low-rank continuation
  const void* A2;
  const void* B2;
  int64_t a2_sm, a2_sk, b2_sn, b2_sk;
  int32_t K2;
  // block-sparse
  int32_t bs_mode, bs_block, bs_nnz;
  const int32_t* bs_index;  // int32 pairs
  const int32_t* bs_count;  // entries per table row, or nullptr (= bs_nnz everywhere)
  int64_t lda, ldb;
};

struct TcParams {
  int32_t num_m_blocks, num_n_blocks;
  int32_t num_k_blocks;   // main reduction, in 64-element units (dense: ceil(K/64); sparse: nnz * block/64)
  int32_t num_k2_blocks;  // low-rank continuation
  // TF32 mode: the reduction axis is cut into k_slices slices of num_k_blocks k-blocks (the last one k_blocks_last);
  // every slice is accumulated in tensor memory on its own and added to D by the epilogue (running fp32 sum)
  int32_t k_slices, k_blocks_last;
  // dense bf16 products with few output tiles and a long reduction: the reduction axis is cut into split_k parts that
  // run as separate tiles (on other SMs) and add their results into a zeroed D (ep.scatter_world = 1); 0 / 1 = off
  int32_t split_k;
  int32_t bs_mode, bs_block, bs_nnz;
  const int32_t* bs_index;  // int32 pairs, see include/leanffn_b200.h
  const int32_t* bs_count;  // entries per table row, or nullptr
  int32_t glu_split;  // > 0: B rows [n, n+128) and [glu_split + n, ...) form one 256-wide tile
  int32_t max_ctas;   // > 0: cap on the persistent grid
  int32_t group_m;    // M-tiles that share one sweep over N in the tile order (0 = kernel default)
  int32_t m_subtiles; // one-CTA kernel: 128-row sub-tiles per CTA tile (1: 128 x N tiles; 2: 256 x 256 or 256 x 128)
  int32_t* status;
  long long wait_limit;  // SM clocks a role waits on an mbarrier before it gives up (0 = the default, about a second)
  EpiParams ep;
};

struct TcOperand {
  const void* ptr;
  int64_t rows;  // extent of the matrix as stored (row-major [rows, cols])
  int64_t cols;
  int64_t ld;
};

int sm_count();
cudaError_t gemm_simt(const SimtOperands& o, const EpiParams& ep, int32_t in_dtype, cudaStream_t st);
int32_t gemm_tcgen05(bool a_mn, bool b_mn, const TcOperand& A, const TcOperand& B, const TcOperand* A2,
                     const TcOperand* B2, TcParams p, int block_n, cudaStream_t st, cudaError_t* cuda_err, bool tf32 = false);
// x [rows, cols] -> out [rows, 3*cols]: per slice of the columns (hi | hi | lo) for role 0, (hi | lo | hi) for role 1
// (see the header).
cudaError_t launch_split_tf32(const float* x, int64_t ldx, float* out, int64_t rows, int64_t cols, int role, int64_t slice,
                              cudaStream_t st);
// partial[0, :] = column sums of x [rows, cols]; partial rows 1 .. ceil(rows/32)-1 are zeroed.
int32_t launch_colsum_into_partials(const void* x, int32_t dtype, int64_t ld, float* partial, int64_t ld_partial,
                                    int64_t rows, int64_t cols, cudaStream_t st);
int32_t launch_peer_barrier(void* const* flags, int32_t rank, int32_t world, int32_t channel, uint32_t epoch,
                            long long limit, int32_t* status, cudaStream_t st);
cudaError_t launch_wait_timeout_probe(int32_t* status, long long limit, cudaStream_t st);
// CTA-pair (cta_group::2) kernel for dense products; tile counts in p are in 256 x 256 tiles.
int32_t gemm_tcgen05_pair(bool a_mn, bool b_mn, const TcOperand& A, const TcOperand& B, const TcOperand* A2,
                          const TcOperand* B2, TcParams p, cudaStream_t st);
int32_t launch_act_fwd(const void* pre, void* hid, int32_t dtype, int64_t rows, int64_t inter, int32_t gated,
                       int32_t act, cudaStream_t st);
int32_t launch_act_bwd(const void* dhid, int64_t ld_dhid, const void* pre, void* dpre, void* hid_out, int32_t dtype,
                       int64_t rows, int64_t inter, int32_t gated, int32_t act, cudaStream_t st);

}  // namespace leanffn
