// GEMM on the Blackwell tensor cores (bf16 operands; fp32 operands multiplied as TF32): TMA tiled loads (each CTA
// fetches its own tiles) stage 128-byte swizzled operand tiles in shared memory, one elected thread issues
// tcgen05.mma with the fp32 accumulator in tensor memory (TMEM), and eight epilogue warps read the accumulator
// back with tcgen05.ld and apply the fused epilogue (bias / gated activation forward and backward / dropout /
// residual / reduce-scatter into peer replicas).  With 128-row tiles the next tile's MMAs already run into the
// other TMEM accumulator stage meanwhile; 256 x 256 tiles fill the whole TMEM and expose the epilogue, but move a
// third less operand data per flop.
//
// One persistent CTA per SM walks a static, M-grouped tile order.  Warp roles:
//   warp 0       TMA producer (one elected lane)
//   warp 1       TMEM allocation + MMA issue (one elected lane)
//   warps 2..9   epilogue; warp w owns TMEM lanes 32*(w%4) .. 32*(w%4)+31, two warps per lane quarter
//                split the tile's 32-column blocks
//
// Operand majorness: a K-major operand is a [rows, K] row-major matrix (TMA box 64 K-elements x 128
// rows); an MN-major operand is a [K, rows] row-major matrix (TMA boxes of 64 rows-elements x 64
// K-rows, one per 64 operand rows).  Both land in the canonical 128B-swizzle UMMA layouts.
//
// Every mbarrier wait is bounded; a role that gives up records a code in the status word, raises a
// CTA-wide abort flag, and all roles drain and free TMEM before returning.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>

#include "gemm_common.cuh"
#include "ptx.cuh"
#include "tc_epilogue.cuh"

namespace leanffn {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 8;
constexpr int TC_THREADS = 64 + 32 * EPI_WARPS;
constexpr int GROUP_M = 16;
constexpr uint32_t A_STAGE_BYTES = BLOCK_M * BLOCK_K * 2;  // 16 KiB
constexpr uint32_t CHUNK_BYTES = 64 * BLOCK_K * 2;         // one MN-major 64 x 64 box, 8 KiB

// MT = number of 128-row accumulator sub-tiles per CTA tile; both sub-tiles share every B stage, which cuts the
// L2 -> shared-memory traffic per flop (by a third for 256-wide tiles, a quarter for 128-wide ones).
//   <256, 1>: 128 x 256 tile, two TMEM accumulator stages (the epilogue of one tile overlaps the MMAs of the next).
//   <256, 2>: 256 x 256 tile; all 512 TMEM columns hold ONE tile, so the epilogue is exposed: long reductions only.
//   <128, 1>: 128 x 128 tile (narrow N, weight-gradient blocks of block-sparse layers), two accumulator stages.
//   <128, 2>: 256 x 128 tile, two accumulator stages of two sub-tiles (512 columns): block-sparse forward / dgrad.
template <int BLOCK_N, int MT = 1>
struct TcConfig {
  static constexpr uint32_t A_BYTES = MT * A_STAGE_BYTES;
  static constexpr uint32_t B_STAGE_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_STAGE_BYTES;
  static constexpr int ACC_STAGES = (MT * BLOCK_N == 512) ? 1 : 2;
  static constexpr uint32_t TMEM_COLS = ACC_STAGES * MT * BLOCK_N;
  static constexpr uint32_t BAR_BYTES = 256;
  static constexpr uint32_t PATCH_BYTES = EPI_WARPS * EPI_PATCH_FLOATS * 4;  // epilogue transposition patches
  static constexpr int STAGES = (227 * 1024 - 1024 - BAR_BYTES - PATCH_BYTES) / STAGE_BYTES;  // 6 / 4 / 4 / 3
  static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + PATCH_BYTES + 1024;  // + alignment slack
};

__device__ __forceinline__ void report(int32_t* status, int32_t code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// TF32: the operands are fp32 (32 elements = 128 bytes per k-block row, K-major only) multiplied as TF32; the byte
// geometry of stages, boxes and descriptors is the same as for bf16.
template <bool A_MN, bool B_MN, int BLOCK_N, int MT, bool TF32 = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                    const TcParams p) {
  using Cfg = TcConfig<BLOCK_N, MT>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ACC_STAGES = Cfg::ACC_STAGES;
  constexpr int TILE_M = BLOCK_M * MT;
  constexpr int KE = TF32 ? BLOCK_K / 2 : BLOCK_K;  // elements per k-block along the reduction axis
  static_assert(!TF32 || (!A_MN && !B_MN), "TF32 operands are K-major");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem ptr, abort
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t abort_slot = tmem_slot + 4;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES + 8u * (2 * STAGES + 4));
  volatile uint32_t* abort_ptr = tmem_slot_ptr + 1;
  (void)abort_slot;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), EPI_WARPS);
    }
    *abort_ptr = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (p.num_k2_blocks > 0) {
      prefetch_tmap(&tmA2);
      prefetch_tmap(&tmB2);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const long long wait_limit = p.wait_limit > 0 ? p.wait_limit : WAIT_LIMIT_CYCLES;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  const int kpb = p.bs_block > 0 ? p.bs_block / BLOCK_K : 1;  // k-blocks per sparse block
  const int sub = p.bs_block >= BLOCK_N ? p.bs_block / BLOCK_N : 1;  // tiles per sparse block along N (and M for wgrad)
  // main k-blocks of a tile: fixed for dense / wgrad, per table row for block-sparse forward / dgrad
  auto main_k_blocks = [&](int n_blk) {
    if ((p.bs_mode == 1 || p.bs_mode == 2) && p.bs_count != nullptr)
      return __ldg(p.bs_count + (p.glu_split > 0 ? n_blk : n_blk / sub)) * kpb;
    return p.num_k_blocks;
  };
  const int group_m = p.group_m > 0 ? p.group_m : GROUP_M;
  const int group_size = group_m * p.num_n_blocks;
  auto tile_coords = [&](int tile, int& m_blk, int& n_blk) {
    const int group = tile / group_size;
    const int first_m = group * group_m;
    const int gm = min(p.num_m_blocks - first_m, group_m);
    const int in_group = tile - group * group_size;
    m_blk = first_m + in_group % gm;
    n_blk = in_group / gm;
  };

  // split-K (dense bf16 only): virtual tile v = part * num_tiles + tile; part s covers k-blocks [s * kps, (s + 1) * kps)
  const int split = (!TF32 && p.split_k > 1) ? p.split_k : 1;
  const int kps = (p.num_k_blocks + split - 1) / split;
  const int num_vtiles = num_tiles * split;
  auto part_k_blocks = [&](int part, int n_blk) {
    return split > 1 ? max(0, min(kps, p.num_k_blocks - part * kps)) : main_k_blocks(n_blk);
  };

  if (warp == 0 && lane == 0) {
    // ------------------------------- TMA producer --------------------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int vtile = blockIdx.x; vtile < num_vtiles && ok; vtile += gridDim.x) {
      const int tile = vtile % num_tiles, part = vtile / num_tiles;
      int m_blk, n_blk;
      tile_coords(tile, m_blk, n_blk);
      const int slices = TF32 ? p.k_slices : 1;
      for (int sl = 0; sl < slices && ok; ++sl) {
      const int kb_main = (TF32 && sl == slices - 1) ? p.k_blocks_last : part_k_blocks(part, n_blk);
      const int kb_base = TF32 ? sl * p.num_k_blocks : part * kps;  // first k-block of this slice / part
      const int kb_total = kb_main + p.num_k2_blocks;
      for (int kb = 0; kb < kb_total; ++kb) {
        if (*abort_ptr != 0 || !mbar_wait_bounded(empty_bar(stage), phase ^ 1u, wait_limit)) {
          report(p.status, LEANFFN_DEV_TIMEOUT_PRODUCER);
          *abort_ptr = 1;
          ok = false;
          break;
        }
        const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
        const uint32_t sb = sa + Cfg::A_BYTES;
        const uint32_t bar = full_bar(stage);
        mbar_arrive_expect_tx(bar, Cfg::STAGE_BYTES);
        const bool second = kb >= kb_main;
        const CUtensorMap* ma = second ? &tmA2 : &tmA;
        const CUtensorMap* mb = second ? &tmB2 : &tmB;
        // coordinates (elements): a_k / b_k along the reduction axis, a_r / b_r along rows
        // gated forward: the 256-wide tile is 128 gate rows (from b_r) + the matching 128 linear rows (from b_r2)
        int a_k, a_r, b_k, b_r, b_r2 = 0, a_r1 = -1;
        if (second) {
          const int k2 = kb - kb_main;
          a_k = b_k = k2 * KE;
          a_r = m_blk * TILE_M;
          b_r = n_blk * BLOCK_N;
          if (p.glu_split > 0) b_r = n_blk * 128, b_r2 = p.glu_split + n_blk * 128;
        } else if (p.bs_mode == 0) {
          a_k = b_k = (kb_base + kb) * KE;
          a_r = m_blk * TILE_M;
          b_r = n_blk * BLOCK_N;
          if (p.glu_split > 0) b_r = n_blk * 128, b_r2 = p.glu_split + n_blk * 128;
        } else if (p.bs_mode == 1 && p.glu_split > 0) {
          // gated block-sparse forward (128-wide blocks): table rows n_blk (gate) and n_blk + I/128 (linear) list the
          // same input blocks, so one A tile meets the weight blocks of both halves
          const int t = kb / kpb, kk = kb - t * kpb;
          const int2* table = reinterpret_cast<const int2*>(p.bs_index);
          const int2 e = __ldg(table + n_blk * p.bs_nnz + t);
          const int2 e2 = __ldg(table + (n_blk + p.glu_split / p.bs_block) * p.bs_nnz + t);
          a_k = e.y * p.bs_block + kk * BLOCK_K;
          a_r = m_blk * TILE_M;
          b_k = kk * BLOCK_K;
          b_r = e.x * p.bs_block;
          b_r2 = e2.x * p.bs_block;
        } else if (p.bs_mode == 1) {
          // table row = output block; entry = (weight block f, input block j)
          const int t = kb / kpb, kk = kb - t * kpb;
          const int2 e = __ldg(reinterpret_cast<const int2*>(p.bs_index) + (n_blk / sub) * p.bs_nnz + t);
          a_k = e.y * p.bs_block + kk * BLOCK_K;
          a_r = m_blk * TILE_M;
          b_k = kk * BLOCK_K;
          b_r = e.x * p.bs_block + (n_blk % sub) * BLOCK_N;
        } else if (p.bs_mode == 2) {
          // table row = input block; entry = (weight block f, output block o); B is read MN-major
          const int t = kb / kpb, kk = kb - t * kpb;
          const int2 e = __ldg(reinterpret_cast<const int2*>(p.bs_index) + (n_blk / sub) * p.bs_nnz + t);
          a_k = e.y * p.bs_block + kk * BLOCK_K;
          a_r = m_blk * TILE_M;
          b_k = e.x * p.bs_block + kk * BLOCK_K;
          b_r = (n_blk % sub) * BLOCK_N;
        } else if (MT == 2) {
          // weight gradient, two 128-wide weight blocks per CTA: blocks 2*m_blk and 2*m_blk + 1 read the same
          // input block (the caller's guarantee), so both sub-tiles share the x stage
          const int2* table = reinterpret_cast<const int2*>(p.bs_index);
          const int2 e = __ldg(table + 2 * m_blk);
          const int2 e1 = __ldg(table + 2 * m_blk + 1);
          a_k = b_k = kb * BLOCK_K;
          a_r = e.x * p.bs_block;
          a_r1 = e1.x * p.bs_block;
          b_r = e.y * p.bs_block + n_blk * BLOCK_N;
        } else {
          // table row = weight block f; entry = (output block o, input block j)
          const int2 e = __ldg(reinterpret_cast<const int2*>(p.bs_index) + m_blk / sub);
          a_k = b_k = kb * BLOCK_K;
          a_r = e.x * p.bs_block + (m_blk % sub) * BLOCK_M;
          b_r = e.y * p.bs_block + n_blk * BLOCK_N;
        }
        if constexpr (A_MN) {
          if (a_r1 < 0) a_r1 = a_r + BLOCK_M;  // second sub-tile: the next 128 rows unless set above
#pragma unroll
          for (int c = 0; c < TILE_M / 64; ++c)
            tma_load_2d(sa + c * CHUNK_BYTES, ma, bar, (c < 2 ? a_r : a_r1 - BLOCK_M) + c * 64, a_k);
        } else {
#pragma unroll
          for (int t = 0; t < MT; ++t) tma_load_2d(sa + t * A_STAGE_BYTES, ma, bar, a_k, a_r + t * BLOCK_M);
        }
        if constexpr (B_MN) {
#pragma unroll
          for (int c = 0; c < BLOCK_N / 64; ++c) tma_load_2d(sb + c * CHUNK_BYTES, mb, bar, b_r + c * 64, b_k);
        } else {
          if (p.glu_split > 0) {
            tma_load_2d(sb, mb, bar, b_k, b_r);
            tma_load_2d(sb + 128 * BLOCK_K * 2, mb, bar, b_k, b_r2);
          } else {
#pragma unroll
            for (int c = 0; c < BLOCK_N / 128; ++c)
              tma_load_2d(sb + c * 128 * BLOCK_K * 2, mb, bar, b_k, b_r + c * 128);
          }
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------- MMA issuer ----------------------------------------------
    constexpr uint32_t idesc = TF32 ? make_idesc_tf32(BLOCK_M, BLOCK_N) : make_idesc_bf16(BLOCK_M, BLOCK_N, A_MN, B_MN);
    constexpr uint64_t a_hi = A_MN ? make_smem_desc_hi(CHUNK_BYTES, 1024) : make_smem_desc_hi(16, 1024);
    constexpr uint64_t b_hi = B_MN ? make_smem_desc_hi(CHUNK_BYTES, 1024) : make_smem_desc_hi(16, 1024);
    constexpr uint32_t a_kstep = A_MN ? 2048u : 32u;  // bytes per UMMA_K step inside a stage
    constexpr uint32_t b_kstep = B_MN ? 2048u : 32u;
    int stage = 0;
    uint32_t phase = 0;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const int mma_slices = TF32 ? p.k_slices : 1;
    for (int vt = 0; ok; ++vt) {  // virtual tiles: (tile, slice) pairs of this CTA, in order
      const int vtile = blockIdx.x + (vt / mma_slices) * gridDim.x, sl = vt % mma_slices;
      if (vtile >= num_vtiles) break;
      const int tile = vtile % num_tiles, part = vtile / num_tiles;
      if (*abort_ptr != 0 || !mbar_wait_bounded(tempty_bar(acc_stage), acc_phase ^ 1u, wait_limit)) {
        report(p.status, LEANFFN_DEV_TIMEOUT_MMA);
        *abort_ptr = 1;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc_stage * (MT * BLOCK_N);
      int m_blk, n_blk;
      tile_coords(tile, m_blk, n_blk);
      const int kb_total = ((TF32 && sl == mma_slices - 1) ? p.k_blocks_last : part_k_blocks(part, n_blk)) + p.num_k2_blocks;
      for (int kb = 0; kb < kb_total; ++kb) {
        if (*abort_ptr != 0 || !mbar_wait_bounded(full_bar(stage), phase, wait_limit)) {
          report(p.status, LEANFFN_DEV_TIMEOUT_MMA);
          *abort_ptr = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
        const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
          const uint64_t db = make_smem_desc(sb + k * b_kstep, b_hi);
#pragma unroll
          for (int t = 0; t < MT; ++t) {  // the sub-tiles read the same B stage
            const uint64_t da = make_smem_desc(sa + t * A_STAGE_BYTES + k * a_kstep, a_hi);
            if constexpr (TF32)
              umma_tf32(d_tmem + t * BLOCK_N, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else
              umma_bf16(d_tmem + t * BLOCK_N, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(empty_bar(stage));  // frees the smem stage once these MMAs have read it
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      umma_commit(tfull_bar(acc_stage));  // accumulator complete
      if (++acc_stage == ACC_STAGES) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  } else if (warp >= 2) {
    // ------------------------------- epilogue ------------------------------------------------
    const EpiParams& ep = p.ep;
    const int quarter = warp & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float* patch = reinterpret_cast<float*>(smem_gen + STAGES * Cfg::STAGE_BYTES + Cfg::BAR_BYTES) +
                   (warp - 2) * EPI_PATCH_FLOATS;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    // TF32 mode, slices after the first: no bias, and the running sum already in D is added (every element of D is
    // written and read back by the same thread, so program order makes the earlier store visible)
    EpiParams ep_sum = ep;
    if constexpr (TF32) {
      ep_sum.bias = nullptr;
      ep_sum.aux = ep.D, ep_sum.ldaux = ep.ldd, ep_sum.aux_dtype = LEANFFN_F32;
    }
    const int epi_slices = TF32 ? p.k_slices : 1;
    bool alive = true;
    for (int vtile = blockIdx.x; vtile < num_vtiles && alive; vtile += gridDim.x) {
      const int tile = vtile % num_tiles, part = vtile / num_tiles;
      int m_blk, n_blk;
      tile_coords(tile, m_blk, n_blk);
#pragma unroll 1
      for (int t = 0; t < MT; ++t)
        epilogue_prefetch_aux<BLOCK_N>(ep, static_cast<int64_t>(m_blk) * TILE_M + t * BLOCK_M + quarter * 32, n_blk, lane,
                                       (warp - 2) >> 2, 2);
      for (int sl = 0; sl < epi_slices; ++sl) {
      if (*abort_ptr != 0 || !mbar_wait_bounded(tfull_bar(acc_stage), acc_phase, wait_limit)) {
        report(p.status, LEANFFN_DEV_TIMEOUT_EPILOGUE);
        *abort_ptr = 1;
        alive = false;
        break;
      }
      tc_fence_after();
      const bool acc_valid = part_k_blocks(part, n_blk) + p.num_k2_blocks > 0;  // empty reduction: acc is all zeros
#pragma unroll 1
      for (int t = 0; t < MT; ++t) {
        const int64_t row0 = static_cast<int64_t>(m_blk) * TILE_M + t * BLOCK_M + quarter * 32;
        const uint32_t t_acc = tmem_base + lane_addr + (acc_stage * MT + t) * BLOCK_N;
        epilogue_tile<BLOCK_N>((TF32 && sl > 0) ? ep_sum : ep, p.glu_split, t_acc, row0, n_blk, acc_valid, patch, lane,
                               (warp - 2) >> 2, 2);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc_stage));
      if (++acc_stage == ACC_STAGES) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
      }
    }
    if (ep.scatter_world > 0) __threadfence_system();  // contributions to peer replicas are out before the kernel ends
  }

  // ------------------------------- teardown ------------------------------------------------------
  __syncwarp();
  if (*abort_ptr != 0) {
    // let copies that may still be in flight land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// One thread waits, with the given limit, on an mbarrier that nobody ever arrives at: the wait must give up, record
// its code in the status word and return, exactly as the roles of the GEMM kernel do when a peer role stalls.
__global__ void wait_timeout_probe_kernel(int32_t* status, long long limit) {
  __shared__ alignas(8) uint64_t bar;
  const uint32_t addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(addr, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !mbar_wait_bounded(addr, 0u, limit)) report(status, LEANFFN_DEV_TIMEOUT_EPILOGUE);
}

cudaError_t launch_wait_timeout_probe(int32_t* status, long long limit, cudaStream_t st) {
  wait_timeout_probe_kernel<<<1, 32, 0, st>>>(status, limit);
  return cudaGetLastError();
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  // cuTensorMapEncodeTiled is a driver call and needs a current context on the calling thread.  A thread that has
  // made no context-binding runtime call yet (an autograd worker whose first operation is this one) has none and the
  // encoder answers CUDA_ERROR_INVALID_CONTEXT: bind the device's primary context once per thread.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension ld (elements);
// box = box_cols (inner, 64 elements = 128 bytes) x box_rows, 128-byte swizzle, zero fill out of bounds.
bool make_tmap_bf16(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, uint32_t box_cols,
                    uint32_t box_rows, bool fp32 = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * (fp32 ? 4 : 2)};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(out, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
            dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 4D bf16 tensor map over a [batch, len, heads, head_dim] view: element (b, s, h, x) lies at
// base + ((b * len + s) * ld + h * head_dim + x) * 2 bytes.  Box = 64 x 1 x box_rows x 1 (head_dim, head, rows, batch),
// 128-byte swizzle; columns beyond head_dim and rows beyond len read as zero.
bool make_tmap_bf16_heads(CUtensorMap* out, const void* base, int64_t batch, int64_t len, int64_t heads,
                          int64_t head_dim, int64_t ld, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(len), static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(ld) * 2,
                                 static_cast<cuuint64_t>(len) * static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS && getenv("LEANFFN_DEBUG") != nullptr)
    fprintf(stderr, "leanffn: cuTensorMapEncodeTiled failed (%d): base %p dims %llu %llu %llu %llu strides %llu %llu %llu\n",
            static_cast<int>(r), base, (unsigned long long)dims[0], (unsigned long long)dims[1],
            (unsigned long long)dims[2], (unsigned long long)dims[3], (unsigned long long)strides[0],
            (unsigned long long)strides[1], (unsigned long long)strides[2]);
  return r == CUDA_SUCCESS;
}

// 4D fp32 tensor map over a contiguous [batch, len, heads, head_dim] tensor for TMA reductions of [128 rows x 32
// columns] boxes (128 bytes per row, 128-byte swizzle in shared memory); rows beyond len and columns beyond head_dim
// are clipped.
bool make_tmap_f32_heads(CUtensorMap* out, void* base, int64_t batch, int64_t len, int64_t heads, int64_t head_dim) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(len), static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(head_dim) * 4, static_cast<cuuint64_t>(heads * head_dim) * 4,
                                 static_cast<cuuint64_t>(len) * static_cast<cuuint64_t>(heads * head_dim) * 4};
  const cuuint32_t box[4] = {32, 1, 128, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN, int BLOCK_N, int MT, bool TF32 = false>
static cudaError_t tc_launch_t(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& a2,
                               const CUtensorMap& b2, const TcParams& p, cudaStream_t st) {
  using Cfg = TcConfig<BLOCK_N, MT>;
  auto kern = gemm_tcgen05_kernel<A_MN, B_MN, BLOCK_N, MT, TF32>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int tiles = p.num_m_blocks * p.num_n_blocks * (p.split_k > 1 ? p.split_k : 1);
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (p.max_ctas > 0 && grid > p.max_ctas) grid = p.max_ctas;
  kern<<<grid, TC_THREADS, Cfg::SMEM_BYTES, st>>>(a, b, a2, b2, p);
  return cudaGetLastError();
}

// Returns LEANFFN_OK, or a negative code when the problem does not fit the tensor-core kernel's
// constraints (the caller then uses the SIMT kernel).
int32_t gemm_tcgen05(bool a_mn, bool b_mn, const TcOperand& A, const TcOperand& B, const TcOperand* A2,
                     const TcOperand* B2, TcParams p, int block_n, cudaStream_t st, cudaError_t* cuda_err, bool tf32) {
  *cuda_err = cudaSuccess;
  CUtensorMap ta, tb, ta2, tb2;
  auto encode = [&](CUtensorMap* m, const TcOperand& o, bool mn) {
    if (tf32) return make_tmap_bf16(m, o.ptr, o.rows, o.cols, o.ld, 32, 128, true);
    return make_tmap_bf16(m, o.ptr, o.rows, o.cols, o.ld, 64, mn ? 64 : 128, false);
  };
  if (!encode(&ta, A, a_mn) || !encode(&tb, B, b_mn)) return LEANFFN_ERR_DRIVER;
  if (A2 != nullptr && B2 != nullptr) {
    if (!encode(&ta2, *A2, a_mn) || !encode(&tb2, *B2, b_mn)) return LEANFFN_ERR_DRIVER;
  } else {
    ta2 = ta;
    tb2 = tb;
  }
  cudaError_t e;
#define TC_GO(AM, BM, BN) e = tc_launch_t<AM, BM, BN, 1>(ta, tb, ta2, tb2, p, st)
  if (tf32) {
    if (a_mn || b_mn || p.m_subtiles != 1) return LEANFFN_ERR_UNSUPPORTED;
    if (block_n == 256) e = tc_launch_t<false, false, 256, 1, true>(ta, tb, ta2, tb2, p, st);
    else e = tc_launch_t<false, false, 128, 1, true>(ta, tb, ta2, tb2, p, st);
  } else if (block_n == 128 && p.m_subtiles == 2) {
    if (!a_mn && !b_mn) e = tc_launch_t<false, false, 128, 2>(ta, tb, ta2, tb2, p, st);
    else if (!a_mn && b_mn) e = tc_launch_t<false, true, 128, 2>(ta, tb, ta2, tb2, p, st);
    else if (a_mn && b_mn) e = tc_launch_t<true, true, 128, 2>(ta, tb, ta2, tb2, p, st);
    else return LEANFFN_ERR_UNSUPPORTED;
  } else if (block_n == 256 && p.m_subtiles == 2) {
    if (!a_mn && !b_mn) e = tc_launch_t<false, false, 256, 2>(ta, tb, ta2, tb2, p, st);
    else if (!a_mn && b_mn) e = tc_launch_t<false, true, 256, 2>(ta, tb, ta2, tb2, p, st);
    else if (a_mn && b_mn) e = tc_launch_t<true, true, 256, 2>(ta, tb, ta2, tb2, p, st);
    else return LEANFFN_ERR_UNSUPPORTED;
  } else if (block_n == 256) {
    if (!a_mn && !b_mn) TC_GO(false, false, 256);
    else if (!a_mn && b_mn) TC_GO(false, true, 256);
    else if (a_mn && b_mn) TC_GO(true, true, 256);
    else return LEANFFN_ERR_UNSUPPORTED;
  } else {
    if (!a_mn && !b_mn) TC_GO(false, false, 128);
    else if (!a_mn && b_mn) TC_GO(false, true, 128);
    else if (a_mn && b_mn) TC_GO(true, true, 128);
    else return LEANFFN_ERR_UNSUPPORTED;
  }
#undef TC_GO
  *cuda_err = e;
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}

}  // namespace leanffn


