// C-ABI GEMM entry point: validates the descriptor, picks the tcgen05 tensor-core kernel when the
// problem meets its layout rules (bf16 operands, 16-byte aligned pitches, block-sparse blocks that are
// multiples of 128) and the SIMT kernel otherwise.  There is no host or library fallback: both paths
// are this library's own device code.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "gemm_common.cuh"
#include "nvtx_range.cuh"

namespace leanffn {

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline size_t esize(int32_t dtype) { return dtype == LEANFFN_BF16 ? 2 : 4; }
static inline bool pitch16(int64_t ld, int32_t dtype) { return (ld * static_cast<int64_t>(esize(dtype))) % 16 == 0; }

}  // namespace leanffn

using namespace leanffn;

extern "C" int32_t leanffn_abi_version(void) { return LEANFFN_ABI_VERSION; }

extern "C" const char* leanffn_status_string(int32_t s) {
  switch (s) {
    case LEANFFN_OK: return "ok";
    case LEANFFN_ERR_NULL: return "null pointer argument";
    case LEANFFN_ERR_SHAPE: return "invalid shape";
    case LEANFFN_ERR_ALIGN: return "pointer or pitch not aligned";
    case LEANFFN_ERR_DTYPE: return "unsupported element type combination";
    case LEANFFN_ERR_UNSUPPORTED: return "unsupported option";
    case LEANFFN_ERR_DRIVER: return "cuTensorMapEncodeTiled unavailable or failed";
    case LEANFFN_ERR_TOO_LARGE: return "size beyond the supported maximum";
    default: break;
  }
  if (s >= 1000) return cudaGetErrorString(static_cast<cudaError_t>(s - 1000));
  return "unknown status";
}

// ---- timing of GEMM launches ------------------------------------------------------------------------------
namespace {
struct GemmTimer {
  int32_t capacity;
  int32_t timed;
  int32_t dropped;
  cudaEvent_t* events;  // 2 per slot
  double* flops;
};
}  // namespace

extern "C" int32_t leanffn_timer_create(int32_t capacity, void** timer) {
  if (timer == nullptr) return LEANFFN_ERR_NULL;
  if (capacity <= 0 || capacity > (1 << 20)) return LEANFFN_ERR_SHAPE;
  GemmTimer* t = new GemmTimer{capacity, 0, 0, new cudaEvent_t[2 * static_cast<size_t>(capacity)], new double[capacity]};
  for (int32_t i = 0; i < 2 * capacity; ++i) {
    const cudaError_t e = cudaEventCreate(&t->events[i]);
    if (e != cudaSuccess) {
      for (int32_t j = 0; j < i; ++j) cudaEventDestroy(t->events[j]);
      delete[] t->events;
      delete[] t->flops;
      delete t;
      return 1000 + static_cast<int32_t>(e);
    }
  }
  *timer = t;
  return LEANFFN_OK;
}

extern "C" int32_t leanffn_timer_reset(void* timer) {
  if (timer == nullptr) return LEANFFN_ERR_NULL;
  GemmTimer* t = static_cast<GemmTimer*>(timer);
  t->timed = t->dropped = 0;
  return LEANFFN_OK;
}

extern "C" int32_t leanffn_timer_summary(void* timer, double* flops, double* seconds, int32_t* timed_launches,
                                         int32_t* dropped_launches) {
  if (timer == nullptr) return LEANFFN_ERR_NULL;
  GemmTimer* t = static_cast<GemmTimer*>(timer);
  double f = 0.0, s = 0.0;
  for (int32_t i = 0; i < t->timed; ++i) {
    cudaError_t e = cudaEventSynchronize(t->events[2 * i + 1]);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t->events[2 * i], t->events[2 * i + 1]);
    if (e != cudaSuccess) return 1000 + static_cast<int32_t>(e);
    f += t->flops[i];
    s += 1e-3 * static_cast<double>(ms);
  }
  if (flops != nullptr) *flops = f;
  if (seconds != nullptr) *seconds = s;
  if (timed_launches != nullptr) *timed_launches = t->timed;
  if (dropped_launches != nullptr) *dropped_launches = t->dropped;
  return LEANFFN_OK;
}

extern "C" int32_t leanffn_timer_destroy(void* timer) {
  if (timer == nullptr) return LEANFFN_OK;
  GemmTimer* t = static_cast<GemmTimer*>(timer);
  for (int32_t i = 0; i < 2 * t->capacity; ++i) cudaEventDestroy(t->events[i]);
  delete[] t->events;
  delete[] t->flops;
  delete t;
  return LEANFFN_OK;
}

static int32_t gemm_impl(const leanffn_gemm_desc* d, void* stream);

extern "C" int32_t leanffn_gemm(const leanffn_gemm_desc* d, void* stream) {
  if (d == nullptr) return LEANFFN_ERR_NULL;
  static const char* const kNames[6] = {"leanffn_gemm store", "leanffn_gemm glu_fwd", "leanffn_gemm act_fwd",
                                        "leanffn_gemm dropout_residual", "leanffn_gemm glu_bwd", "leanffn_gemm act_bwd"};
  NvtxRange range(d->epilogue >= 0 && d->epilogue < 6 ? kNames[d->epilogue] : "leanffn_gemm");
  GemmTimer* t = static_cast<GemmTimer*>(d->timer);
  int32_t slot = -1;
  if (t != nullptr && d->M > 0) {
    if (t->timed < t->capacity) {
      slot = t->timed;
      cudaEventRecord(t->events[2 * slot], static_cast<cudaStream_t>(stream));
    } else {
      ++t->dropped;
    }
  }
  const int32_t status = gemm_impl(d, stream);
  if (slot >= 0) {
    cudaEventRecord(t->events[2 * slot + 1], static_cast<cudaStream_t>(stream));
    if (status == LEANFFN_OK) {
      double k = d->K;
      if (d->bs_mode == 1 || d->bs_mode == 2) k = static_cast<double>(d->bs_nnz) * d->bs_block;
      if (d->in_dtype == LEANFFN_TF32) k /= 3.0;  // three TF32 products stand for one fp32 product
      t->flops[slot] = 2.0 * d->M * static_cast<double>(d->N) * (k + d->K2);
      ++t->timed;
    }
  }
  return status;
}

static int32_t gemm_impl(const leanffn_gemm_desc* d, void* stream) {
  if (d == nullptr) return LEANFFN_ERR_NULL;
  if (d->M < 0 || d->N <= 0 || d->K <= 0 || d->K2 < 0) return LEANFFN_ERR_SHAPE;
  if (d->M > 0 && (d->A == nullptr || d->B == nullptr || d->D == nullptr)) return LEANFFN_ERR_NULL;
  if (d->in_dtype != LEANFFN_F32 && d->in_dtype != LEANFFN_BF16 && d->in_dtype != LEANFFN_TF32) return LEANFFN_ERR_DTYPE;
  if (d->d_dtype != LEANFFN_F32 && d->d_dtype != LEANFFN_BF16) return LEANFFN_ERR_DTYPE;
  if (d->epilogue < LEANFFN_EPI_STORE || d->epilogue > LEANFFN_EPI_ACT_BWD) return LEANFFN_ERR_UNSUPPORTED;
  if (d->act < 0 || d->act >= LEANFFN_ACT_COUNT) return LEANFFN_ERR_UNSUPPORTED;
  if (d->bs_mode < 0 || d->bs_mode > 3) return LEANFFN_ERR_UNSUPPORTED;
  if (!(d->dropout_p >= 0.f && d->dropout_p < 1.f)) return LEANFFN_ERR_UNSUPPORTED;
  if (d->wait_limit_cycles < 0 || d->tf32_k_slice < 0) return LEANFFN_ERR_UNSUPPORTED;
  if (d->K2 > 0 && (d->A2 == nullptr || d->B2 == nullptr)) return LEANFFN_ERR_NULL;
  const int epi = d->epilogue;
  const bool needs_d2 = epi == LEANFFN_EPI_GLU_FWD || epi == LEANFFN_EPI_ACT_FWD;
  const bool needs_aux = epi == LEANFFN_EPI_GLU_BWD || epi == LEANFFN_EPI_ACT_BWD;
  if (needs_d2 && d->D2 == nullptr) return LEANFFN_ERR_NULL;
  if (needs_aux && d->aux == nullptr) return LEANFFN_ERR_NULL;
  if (epi == LEANFFN_EPI_GLU_FWD && (d->N % 2 != 0)) return LEANFFN_ERR_SHAPE;
  if (d->bs_mode != 0) {
    if (d->bs_index == nullptr) return LEANFFN_ERR_NULL;
    if (d->bs_block <= 0 || d->bs_nnz <= 0 || d->bs_num_blocks <= 0) return LEANFFN_ERR_SHAPE;
    if (d->bs_mode == 3) {
      if (!d->a_mn_major || !d->b_mn_major || d->N != d->bs_block ||
          d->M != static_cast<int64_t>(d->bs_num_blocks) * d->bs_block || d->K2 != 0 || d->bs_nnz != 1)
        return LEANFFN_ERR_SHAPE;
    } else {
      if (d->a_mn_major || d->N % d->bs_block != 0 || d->K % d->bs_block != 0) return LEANFFN_ERR_SHAPE;
    }
    const bool bwd_epilogue = epi == LEANFFN_EPI_GLU_BWD || epi == LEANFFN_EPI_ACT_BWD;
    const bool fwd_epilogue = epi == LEANFFN_EPI_DROPOUT_RESIDUAL || epi == LEANFFN_EPI_GLU_FWD;
    if (epi != LEANFFN_EPI_STORE && !(d->bs_mode == 2 && bwd_epilogue) && !(d->bs_mode == 1 && fwd_epilogue))
      return LEANFFN_ERR_UNSUPPORTED;
    // gated forward: one tile = a gate block and its linear partner, which must share their input blocks
    if (epi == LEANFFN_EPI_GLU_FWD && (d->bs_block != 128 || (d->N / 2) % 128 != 0 || d->in_dtype != LEANFFN_BF16))
      return LEANFFN_ERR_UNSUPPORTED;
  }
  if (d->scatter_world != 0) {
    if (d->scatter_world < 0 || d->scatter_world > 8) return LEANFFN_ERR_TOO_LARGE;
    if (epi != LEANFFN_EPI_STORE || d->bias != nullptr || d->scatter_block_shift < 7 || d->scatter_block_shift > 30)
      return LEANFFN_ERR_UNSUPPORTED;
    for (int k = 0; k < d->scatter_world; ++k) {
      if (d->scatter_D[k] == nullptr) return LEANFFN_ERR_NULL;
      if (!aligned16(d->scatter_D[k])) return LEANFFN_ERR_ALIGN;
    }
  }
  if (d->colsum_partial != nullptr) {
    if (!needs_aux) return LEANFFN_ERR_UNSUPPORTED;  // activation-backward epilogues only
    const int64_t width = epi == LEANFFN_EPI_GLU_BWD ? 2 * static_cast<int64_t>(d->N) : d->N;
    if (d->ld_colsum < width || d->ld_colsum % 2 != 0) return LEANFFN_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(d->colsum_partial) % 8 != 0) return LEANFFN_ERR_ALIGN;
  }
  if (d->M == 0) return LEANFFN_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  EpiParams ep{};
  ep.kind = epi;
  ep.act = d->act;
  ep.M = d->M;
  ep.N = d->N;
  ep.D = d->D;
  ep.ldd = d->ldd;
  ep.d_dtype = d->d_dtype;
  ep.D2 = d->D2;
  ep.ldd2 = d->ldd2;
  ep.bias = d->bias;
  ep.bias_dtype = d->bias_dtype;
  ep.aux = d->aux;
  ep.ldaux = d->ldaux;
  ep.aux_dtype = d->aux_dtype;
  ep.threshold = d->dropout_p > 0.f ? dropout_threshold(d->dropout_p) : 0u;
  ep.keep_scale = 1.0f / (1.0f - d->dropout_p);
  ep.seed = d->seed;
  ep.elem_offset = d->elem_offset;
  ep.scatter_world = d->scatter_world;
  ep.scatter_shift = d->scatter_block_shift;
  for (int k = 0; k < 8; ++k) ep.scatter_D[k] = k < d->scatter_world ? d->scatter_D[k] : nullptr;
  ep.colsum = d->colsum_partial;
  ep.ldcolsum = d->ld_colsum;
#ifdef LEANFFN_ABLATE_RUNTIME
  {
    const char* v = getenv("LEANFFN_ABLATE");  // read on every call: the measurement script changes it between runs
    ep.ablate = v != nullptr ? atoi(v) : 0;
  }
#endif

  // ---- fp32 operands on the tensor cores (TF32 multiplication) ---------------------------------------
  if (d->in_dtype == LEANFFN_TF32) {
    if (d->a_mn_major || d->b_mn_major || d->bs_mode != 0 || d->K2 != 0 || epi != LEANFFN_EPI_STORE ||
        d->d_dtype != LEANFFN_F32 || d->scatter_world != 0 || d->M < 64 || d->N < 64 || d->K < 32 || d->N % 8 != 0)
      return LEANFFN_ERR_UNSUPPORTED;
    if (!aligned16(d->A) || !aligned16(d->B) || !aligned16(d->D) || !pitch16(d->lda, LEANFFN_F32) ||
        !pitch16(d->ldb, LEANFFN_F32) || !pitch16(d->ldd, LEANFFN_F32) || (d->bias != nullptr && !aligned16(d->bias)))
      return LEANFFN_ERR_ALIGN;
    if (d->aux != nullptr && (d->aux_dtype != LEANFFN_F32 || !aligned16(d->aux) || !pitch16(d->ldaux, LEANFFN_F32)))
      return LEANFFN_ERR_ALIGN;
    TcParams p{};
    p.ep = ep;
    p.status = d->status_word;
    p.wait_limit = d->wait_limit_cycles;
    p.max_ctas = d->max_ctas;
    p.m_subtiles = 1;
    const int block_n = d->N <= 128 ? 128 : 256;
    p.num_m_blocks = static_cast<int32_t>((d->M + 127) / 128);
    p.num_n_blocks = static_cast<int32_t>((d->N + block_n - 1) / block_n);
    p.num_k_blocks = static_cast<int32_t>((d->K + 31) / 32);
    p.k_slices = 1;
    p.k_blocks_last = p.num_k_blocks;
    if (d->tf32_k_slice > 0) {
      // slices of tf32_k_slice elements of the (tripled) reduction axis, the last one takes the remainder: the rule
      // leanffn_split_tf32 lays the slices out by
      if (d->tf32_k_slice % 96 != 0) return LEANFFN_ERR_SHAPE;  // 3 parts of a multiple of 32 elements (one k-block)
      const int32_t slices = d->K / d->tf32_k_slice > 0 ? d->K / d->tf32_k_slice : 1;
      p.k_slices = slices;
      p.num_k_blocks = d->tf32_k_slice / 32;
      p.k_blocks_last = static_cast<int32_t>((d->K - static_cast<int64_t>(slices - 1) * d->tf32_k_slice + 31) / 32);
      if (slices > 1 && d->aux != nullptr) return LEANFFN_ERR_UNSUPPORTED;  // the running sum lives in D itself
    }
    TcOperand A{}, B{};
    A.ptr = d->A, A.ld = d->lda, A.rows = d->M, A.cols = d->K;
    B.ptr = d->B, B.ld = d->ldb, B.rows = d->N, B.cols = d->K;
    cudaError_t ce;
    return gemm_tcgen05(false, false, A, B, nullptr, nullptr, p, block_n, st, &ce, true);
  }

  // Reduction length seen by the kernels.
  int64_t k_eff = d->K;
  if (d->bs_mode == 1 || d->bs_mode == 2) k_eff = static_cast<int64_t>(d->bs_nnz) * d->bs_block;

  // ---- tensor-core path ------------------------------------------------------------------------
  bool tc = d->in_dtype == LEANFFN_BF16 && !d->force_simt;
  tc = tc && d->M >= 64 && d->N >= 64 && k_eff >= 32;
  tc = tc && aligned16(d->A) && aligned16(d->B) && pitch16(d->lda, LEANFFN_BF16) && aligned16(d->D) &&
       pitch16(d->ldd, d->d_dtype) && d->N % 8 == 0;
  if (d->bs_mode == 0 || d->bs_mode == 3) tc = tc && pitch16(d->ldb, LEANFFN_BF16);
  if (d->bs_mode != 0) tc = tc && d->bs_block % 128 == 0;
  if (d->a_mn_major && !d->b_mn_major) tc = false;  // combination not used by any caller
  if (d->K2 > 0)
    tc = tc && aligned16(d->A2) && aligned16(d->B2) && pitch16(d->lda2, LEANFFN_BF16) && pitch16(d->ldb2, LEANFFN_BF16);
  if (d->bias != nullptr) tc = tc && aligned16(d->bias);
  if (d->aux != nullptr) tc = tc && aligned16(d->aux) && pitch16(d->ldaux, d->aux_dtype) &&
              (d->aux_dtype == LEANFFN_BF16 || epi == LEANFFN_EPI_DROPOUT_RESIDUAL);
  if (d->D2 != nullptr) tc = tc && aligned16(d->D2) && pitch16(d->ldd2, d->d_dtype);
  if (needs_d2) tc = tc && d->d_dtype == LEANFFN_BF16;
  if (epi == LEANFFN_EPI_GLU_FWD) tc = tc && (d->N / 2) % 8 == 0 && (d->bs_mode == 0 || d->bs_mode == 1);
  if (ep.threshold != 0u) tc = tc && d->elem_offset % 4 == 0;

  if (tc) {
    TcParams p{};
    p.ep = ep;
    p.status = d->status_word;
    p.wait_limit = d->wait_limit_cycles;
    p.bs_mode = d->bs_mode;
    p.bs_block = d->bs_mode ? d->bs_block : 0;
    p.bs_nnz = d->bs_nnz;
    p.bs_index = d->bs_index;
    p.bs_count = d->bs_count;
    p.glu_split = 0;
    p.max_ctas = d->max_ctas;
    int block_n = (d->bs_mode != 0 || d->N <= 128) ? 128 : 256;
    int64_t n_tiles_n;
    if (epi == LEANFFN_EPI_GLU_FWD) {
      block_n = 256;
      p.glu_split = d->N / 2;
      n_tiles_n = (p.glu_split + 127) / 128;
    } else {
      n_tiles_n = (d->N + block_n - 1) / block_n;
    }
    p.num_m_blocks = static_cast<int32_t>((d->M + 127) / 128);
    p.num_n_blocks = static_cast<int32_t>(n_tiles_n);
    p.num_k_blocks = static_cast<int32_t>((k_eff + 63) / 64);
    p.num_k2_blocks = static_cast<int32_t>((d->K2 + 63) / 64);
    p.k_slices = 1;
    p.k_blocks_last = p.num_k_blocks;
    TcOperand A{}, B{}, A2{}, B2{};
    A.ptr = d->A;
    A.ld = d->lda;
    B.ptr = d->B;
    B.ld = d->ldb;
    if (d->bs_mode == 0) {
      if (d->a_mn_major) A.rows = d->K, A.cols = d->M; else A.rows = d->M, A.cols = d->K;
      if (d->b_mn_major) B.rows = d->K, B.cols = d->N; else B.rows = d->N, B.cols = d->K;
    } else if (d->bs_mode == 1 || d->bs_mode == 2) {
      // A: activations [M, K]; B: the weight blocks seen as one [(num_blocks * block), block] matrix
      A.rows = d->M, A.cols = d->K;
      B.rows = static_cast<int64_t>(d->bs_num_blocks) * d->bs_block;
      B.cols = d->bs_block;
      B.ld = d->bs_block;
    } else {
      A.rows = d->K, A.cols = d->lda;  // dy [tokens, out_features]
      B.rows = d->K, B.cols = d->ldb;  // x  [tokens, in_features]
    }
    if (d->K2 > 0) {
      A2.ptr = d->A2, A2.ld = d->lda2;
      B2.ptr = d->B2, B2.ld = d->ldb2;
      if (d->a_mn_major) A2.rows = d->K2, A2.cols = d->M; else A2.rows = d->M, A2.cols = d->K2;
      if (d->b_mn_major) B2.rows = d->K2, B2.cols = d->N; else B2.rows = d->N, B2.cols = d->K2;
    }
    static const int tile_override = []() {
      const char* v = getenv("LEANFFN_GEMM_TILE");
      return v != nullptr ? atoi(v) : 0;
    }();
    static const int group_override = []() {
      const char* v = getenv("LEANFFN_GROUP_M");
      return v != nullptr ? atoi(v) : 0;
    }();
    p.group_m = group_override;
    // Dense products with at least one full 256 x 256 tile can run on CTA pairs (cta_group::2).  Under the
    // 1 kW power cap of long runs the one-CTA kernel sustains the higher rate, so it is the default;
    // LEANFFN_GEMM_KERNEL=pair selects the CTA-pair kernel (it wins on short, cool bursts).
    static const bool pair_enabled = []() {
      const char* v = getenv("LEANFFN_GEMM_KERNEL");
      return v != nullptr && strcmp(v, "pair") == 0;
    }();
    if (pair_enabled && d->bs_mode == 0 && block_n == 256 && d->M > 128 && d->scatter_world == 0) {
      p.num_m_blocks = static_cast<int32_t>((d->M + 255) / 256);
      return gemm_tcgen05_pair(d->a_mn_major != 0, d->b_mn_major != 0, A, B, d->K2 > 0 ? &A2 : nullptr,
                               d->K2 > 0 ? &B2 : nullptr, p, st);
    }
    // Long reductions run 256 x 256 tiles per CTA (two accumulator sub-tiles sharing each B stage): a third less
    // operand traffic per flop; the exposed epilogue is a few percent of such a tile.  LEANFFN_GEMM_TILE=128 / 256
    // forces one or the other.
    p.m_subtiles = 1;
    if (d->bs_mode == 0 && block_n == 256 && d->M >= 256) {
      const int64_t k_total = k_eff + d->K2;
      // wave efficiency of a persistent grid: tiles / (waves * SMs); the larger tile must not quantise worse
      const int sms = sm_count();
      auto wave_eff = [sms](int64_t tiles) {
        return static_cast<double>(tiles) / static_cast<double>(((tiles + sms - 1) / sms) * sms);
      };
      const int64_t tiles128 = static_cast<int64_t>(p.num_m_blocks) * p.num_n_blocks;
      const int64_t tiles256 = ((d->M + 255) / 256) * static_cast<int64_t>(p.num_n_blocks);
      const bool pays = k_total >= 4096 && wave_eff(tiles256) >= wave_eff(tiles128) - 0.05;
      if (tile_override == 256 || (tile_override == 0 && pays)) {
        p.m_subtiles = 2;
        p.num_m_blocks = static_cast<int32_t>((d->M + 255) / 256);
        if (p.group_m == 0) p.group_m = 8;  // 8 x 256 rows per sweep: measured best for the 256 x 256 tiles
      }
    }
    if ((d->bs_mode == 1 || d->bs_mode == 2) && block_n == 128 && d->M >= 256 && tile_override != 128) {
      // block-sparse forward / input gradient: every weight block meets two 128-token sub-tiles per CTA
      // (256 x 128 tile, the accumulators stay double-buffered), a quarter less operand traffic per flop
      const int sms = sm_count();
      auto wave_eff = [sms](int64_t tiles) {
        return static_cast<double>(tiles) / static_cast<double>(((tiles + sms - 1) / sms) * sms);
      };
      const int64_t tiles128 = static_cast<int64_t>(p.num_m_blocks) * p.num_n_blocks;
      const int64_t tiles256 = ((d->M + 255) / 256) * static_cast<int64_t>(p.num_n_blocks);
      if (tile_override == 256 || wave_eff(tiles256) >= wave_eff(tiles128) - 0.05) {
        p.m_subtiles = 2;
        p.num_m_blocks = static_cast<int32_t>((d->M + 255) / 256);
        if (p.group_m == 0) p.group_m = 8;
      }
    }
    if (d->bs_mode == 3 && d->bs_wgrad_pairs != 0 && d->bs_block == 128 && d->bs_num_blocks % 2 == 0 &&
        tile_override != 128) {
      p.m_subtiles = 2;  // 256 x 128 tile = two weight blocks that share their x tile
      p.num_m_blocks = d->bs_num_blocks / 2;
    }
    // Split-K: a dense product whose output has fewer 128-row tiles than the device has SMs and whose reduction is
    // long (the weight gradients of narrow layers: [768, 768] from 65 536 tokens is 18 tiles) cuts the reduction into
    // parts that run as tiles of their own and add into a zeroed fp32 result.  LEANFFN_SPLIT_K=1 turns it off.
    p.split_k = 1;
    static const int split_override = []() {
      const char* v = getenv("LEANFFN_SPLIT_K");
      return v != nullptr ? atoi(v) : 0;
    }();
    if (d->bs_mode == 0 && p.m_subtiles == 1 && epi == LEANFFN_EPI_STORE && d->bias == nullptr && d->K2 == 0 &&
        d->scatter_world == 0 && d->d_dtype == LEANFFN_F32 && split_override != 1) {
      const int sms = p.max_ctas > 0 && p.max_ctas < sm_count() ? p.max_ctas : sm_count();
      const int64_t tiles = static_cast<int64_t>(p.num_m_blocks) * p.num_n_blocks;
      auto wave_eff = [sms](int64_t t) {
        return static_cast<double>(t) / static_cast<double>(((t + sms - 1) / sms) * sms);
      };
      int best = 1;
      double best_eff = wave_eff(tiles);
      for (int s = 2; s <= 8; ++s) {
        if (p.num_k_blocks / s < 16) break;  // at least 1024 elements of the reduction per part
        const double e = wave_eff(tiles * s);
        if (e > best_eff + 0.1) best = s, best_eff = e;
      }
      if (split_override > 1 && p.num_k_blocks / split_override >= 1) best = split_override;
      if (best > 1) {
        const cudaError_t me = cudaMemset2DAsync(d->D, static_cast<size_t>(d->ldd) * 4, 0, static_cast<size_t>(d->N) * 4,
                                                 static_cast<size_t>(d->M), st);
        if (me != cudaSuccess) return 1000 + static_cast<int32_t>(me);
        p.split_k = best;
        p.ep.scatter_world = 1;   // the epilogue adds (red.global.add.f32) instead of storing
        p.ep.scatter_shift = 30;
        p.ep.scatter_D[0] = d->D;
      }
    }
    cudaError_t ce;
    return gemm_tcgen05(d->a_mn_major != 0, d->b_mn_major != 0, A, B, d->K2 > 0 ? &A2 : nullptr,
                        d->K2 > 0 ? &B2 : nullptr, p, block_n, st, &ce);
  }

  // ---- SIMT path ---------------------------------------------------------------------------------
  if (d->scatter_world != 0) return LEANFFN_ERR_UNSUPPORTED;  // the scattered reduction exists in the tensor-core kernel only
  SimtOperands o{};
  o.A = d->A;
  o.B = d->B;
  o.lda = d->lda;
  o.ldb = d->ldb;
  o.K = static_cast<int32_t>(k_eff);
  if (d->a_mn_major) o.a_sm = 1, o.a_sk = d->lda; else o.a_sm = d->lda, o.a_sk = 1;
  if (d->b_mn_major) o.b_sn = 1, o.b_sk = d->ldb; else o.b_sn = d->ldb, o.b_sk = 1;
  o.A2 = d->K2 > 0 ? d->A2 : nullptr;
  o.B2 = d->K2 > 0 ? d->B2 : nullptr;
  o.K2 = d->K2;
  if (d->a_mn_major) o.a2_sm = 1, o.a2_sk = d->lda2; else o.a2_sm = d->lda2, o.a2_sk = 1;
  if (d->b_mn_major) o.b2_sn = 1, o.b2_sk = d->ldb2; else o.b2_sn = d->ldb2, o.b2_sk = 1;
  o.bs_mode = d->bs_mode;
  o.bs_block = d->bs_block;
  o.bs_nnz = d->bs_nnz;
  o.bs_index = d->bs_index;
  o.bs_count = d->bs_count;

  cudaError_t e;
  if (epi == LEANFFN_EPI_STORE || epi == LEANFFN_EPI_DROPOUT_RESIDUAL) {
    e = gemm_simt(o, ep, d->in_dtype, st);
    return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
  }
  // Activation epilogues: the product is stored first, the activation runs as a second pass.
  EpiParams plain = ep;
  plain.kind = LEANFFN_EPI_STORE;
  if (epi == LEANFFN_EPI_GLU_FWD || epi == LEANFFN_EPI_ACT_FWD) {
    const bool gated = epi == LEANFFN_EPI_GLU_FWD;
    const int64_t inter = gated ? d->N / 2 : d->N;
    if (d->ldd != d->N || d->ldd2 != inter || inter % 4 != 0) return LEANFFN_ERR_UNSUPPORTED;
    e = gemm_simt(o, plain, d->in_dtype, st);
    if (e != cudaSuccess) return 1000 + static_cast<int32_t>(e);
    return launch_act_fwd(d->D, d->D2, d->d_dtype, d->M, inter, gated ? 1 : 0, d->act, st);
  }
  {
    const bool gated = epi == LEANFFN_EPI_GLU_BWD;
    const int64_t inter = d->N;
    const int64_t ldpre = gated ? 2 * inter : inter;
    if (d->ldd != ldpre || d->ldaux != ldpre || d->aux_dtype != d->d_dtype || inter % 4 != 0)
      return LEANFFN_ERR_UNSUPPORTED;
    if (d->D2 != nullptr && d->ldd2 != inter) return LEANFFN_ERR_UNSUPPORTED;
    // dHid lands in the linear half of dPre (gated) or in dPre itself, then is transformed in place.
    plain.D = static_cast<char*>(d->D) + (gated ? inter * esize(d->d_dtype) : 0);
    plain.bias = nullptr;
    e = gemm_simt(o, plain, d->in_dtype, st);
    if (e != cudaSuccess) return 1000 + static_cast<int32_t>(e);
    const int32_t s = launch_act_bwd(plain.D, ldpre, d->aux, d->D, d->D2, d->d_dtype, d->M, inter, gated ? 1 : 0, d->act, st);
    if (s != LEANFFN_OK || d->colsum_partial == nullptr) return s;
    // same contract as the tensor-core epilogue: the partial rows sum to the column sums of D (row 0 carries them all)
    return launch_colsum_into_partials(d->D, d->d_dtype, ldpre, d->colsum_partial, d->ld_colsum, d->M, ldpre, st);
  }
}

extern "C" int32_t leanffn_selftest_wait_timeout(int32_t* status_word, int64_t limit_cycles, void* stream) {
  if (status_word == nullptr) return LEANFFN_ERR_NULL;
  long long limit = limit_cycles < 1000 ? 1000 : (limit_cycles > 10000000 ? 10000000 : limit_cycles);
  const cudaError_t e = launch_wait_timeout_probe(status_word, limit, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}

extern "C" int32_t leanffn_peer_barrier(void* const* flags, int32_t rank, int32_t world, int32_t channel, uint32_t epoch,
                                        int64_t limit_cycles, int32_t* status_word, void* stream) {
  if (flags == nullptr) return LEANFFN_ERR_NULL;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || channel < 0 || channel >= 4) return LEANFFN_ERR_SHAPE;
  if (limit_cycles < 0) return LEANFFN_ERR_UNSUPPORTED;
  for (int i = 0; i < world; ++i) {
    if (flags[i] == nullptr) return LEANFFN_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(flags[i]) % 4 != 0) return LEANFFN_ERR_ALIGN;
  }
  if (world == 1) return LEANFFN_OK;
  const long long limit = limit_cycles == 0 ? 40000000000LL : limit_cycles;  // ~20 s of SM clocks by default
  return launch_peer_barrier(flags, rank, world, channel, epoch, limit, status_word, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t leanffn_copy_2d(void* dst, uint64_t dst_pitch_bytes, const void* src, uint64_t src_pitch_bytes,
                                   uint64_t width_bytes, uint64_t height, void* stream) {
  if (width_bytes == 0 || height == 0) return LEANFFN_OK;
  if (dst == nullptr || src == nullptr) return LEANFFN_ERR_NULL;
  if (dst_pitch_bytes < width_bytes || src_pitch_bytes < width_bytes) return LEANFFN_ERR_SHAPE;
  const cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch_bytes, src, src_pitch_bytes, width_bytes, height,
                                          cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}

extern "C" int32_t leanffn_split_tf32(const float* x, int64_t ldx, float* out, int64_t rows, int64_t cols, int32_t role,
                                      int64_t slice, void* stream) {
  if (rows < 0 || cols <= 0 || (role != 0 && role != 1) || slice <= 0) return LEANFFN_ERR_SHAPE;
  if (rows == 0) return LEANFFN_OK;
  if (x == nullptr || out == nullptr) return LEANFFN_ERR_NULL;
  const cudaError_t e = launch_split_tf32(x, ldx, out, rows, cols, role, slice, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}
