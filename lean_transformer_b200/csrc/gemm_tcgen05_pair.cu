// bf16 GEMM on CTA pairs: two neighbouring SMs (a thread-block cluster of 2) compute one 256 x 256 output
// tile with tcgen05 cta_group::2.  Each CTA stages its own 128 rows of A and ITS HALF (128 rows) of B with
// its own TMA loads; the tensor cores of both SMs read both halves of B, so every byte of B crosses
// L2 -> shared memory once per pair instead of once per SM.  Per 64-deep k-block a CTA moves 32 KiB for
// 512 tensor-core clocks (64 B/clk/SM), against 96 B/clk/SM for the one-CTA 128 x 256 kernel.
//
// Roles per CTA (320 threads): warp 0 = TMA producer, warp 1 = TMEM allocation (+ MMA issue in the leader CTA,
// rank 0 of the pair), warps 2..9 = epilogue of the CTA's own 128 accumulator rows.
// Synchronisation:
//   full[s]    (leader's shared memory)  both CTAs' TMA bytes are credited to it; the leader's MMA thread waits
//   empty[s]   (each CTA)                the leader's tcgen05.commit arrives on both CTAs' barriers
//   tfull[a]   (each CTA)                accumulator stage a complete: commit arrives on both
//   tempty[a]  (leader's shared memory)  16 arrivals: the 8 epilogue warps of each CTA
// Every wait is bounded; a role that gives up records a code, raises the pair-wide abort flags and all roles
// drain, meet at the closing cluster barrier and free TMEM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "gemm_common.cuh"
#include "ptx.cuh"
#include "tc_epilogue.cuh"

namespace leanffn {

namespace pair {

constexpr int BLOCK_M = 256;       // per pair; 128 per CTA
constexpr int BLOCK_N = 256;       // per pair; each CTA stages 128 rows of B
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int GROUP_M = 8;         // 8 x 256 rows share a sweep over N (L2 reuse of the A panels)
constexpr int MAX_STAGES = 6;
constexpr uint32_t A_BYTES = 128 * BLOCK_K * 2;          // 16 KiB
constexpr uint32_t B_BYTES = 128 * BLOCK_K * 2;          // 16 KiB (this CTA's half)
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;      // 32 KiB
constexpr uint32_t CHUNK_BYTES = 64 * BLOCK_K * 2;       // one MN-major 64 x 64 box
constexpr uint32_t TMEM_COLS = 512;                      // two 256-column accumulator stages
constexpr uint32_t PATCH_BYTES = EPI_WARPS * EPI_PATCH_FLOATS * 4;
constexpr uint32_t SMEM_BYTES = MAX_STAGES * STAGE_BYTES + 256 + PATCH_BYTES + 1024;

}  // namespace pair

__device__ __forceinline__ void report_status(int32_t* status, int32_t code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(pair::THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                         const TcParams p) {
  using namespace pair;
  extern __shared__ uint8_t smem_raw[];
  constexpr int STAGES_ALLOC = MAX_STAGES;
  constexpr int STAGES = MAX_STAGES;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES_ALLOC * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES_ALLOC + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES_ALLOC + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES_ALLOC + 2 + s); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES_ALLOC + 4);
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES_ALLOC * STAGE_BYTES + 8u * (2 * STAGES_ALLOC + 4));
  volatile uint32_t* abort_ptr = tmem_slot_ptr + 1;
  const uint32_t abort_addr = tmem_slot + 4;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 = leader
  const bool leader = rank == 0;
  const uint32_t peer_abort = map_to_cta(abort_addr, rank ^ 1u);
  auto raise_abort = [&](int32_t code) {
    report_status(p.status, code);
    *abort_ptr = 1;
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_abort), "r"(1u) : "memory");
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // the leader producer's arrive.expect_tx (bytes of both CTAs)
      mbar_init(empty_bar(s), 1);  // one commit arrival
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 2 * EPI_WARPS);  // every epilogue warp of both CTAs (used in the leader only)
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
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anything arrives on them remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const int num_pairs = gridDim.x >> 1;
  const int pair_id = blockIdx.x >> 1;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;  // in 256 x 256 tiles
  const int kb_total = p.num_k_blocks + p.num_k2_blocks;
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

  if (warp == 0 && lane == 0) {
    // ------------------------------- TMA producer (both CTAs) ----------------------------------
    const uint32_t leader_full0 = map_to_cta(full_bar(0), 0);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
      int m_blk, n_blk;
      tile_coords(tile, m_blk, n_blk);
      const int a_r = m_blk * BLOCK_M + static_cast<int>(rank) * 128;  // this CTA's rows of A
      // this CTA's 128 rows of B: plain tile, or gate rows (leader) / linear rows (peer) of a gated weight
      const int b_r = p.glu_split > 0 ? (leader ? n_blk * 128 : p.glu_split + n_blk * 128)
                                      : n_blk * BLOCK_N + static_cast<int>(rank) * 128;
      for (int kb = 0; kb < kb_total; ++kb) {
        if (*abort_ptr != 0 || !mbar_wait_bounded(empty_bar(stage), phase ^ 1u)) {
          raise_abort(LEANFFN_DEV_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint32_t sb = sa + A_BYTES;
        const uint32_t bar = leader_full0 + 8u * stage;  // the leader's full barrier, cluster-window address
        if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
        const bool second = kb >= p.num_k_blocks;
        const CUtensorMap* ma = second ? &tmA2 : &tmA;
        const CUtensorMap* mb = second ? &tmB2 : &tmB;
        const int k0 = (second ? kb - p.num_k_blocks : kb) * BLOCK_K;
        if constexpr (A_MN) {
#pragma unroll
          for (int c = 0; c < 2; ++c) tma_load_2d_pair(sa + c * CHUNK_BYTES, ma, bar, a_r + c * 64, k0);
        } else {
          tma_load_2d_pair(sa, ma, bar, k0, a_r);
        }
        if constexpr (B_MN) {
#pragma unroll
          for (int c = 0; c < 2; ++c) tma_load_2d_pair(sb + c * CHUNK_BYTES, mb, bar, b_r + c * 64, k0);
        } else {
          tma_load_2d_pair(sb, mb, bar, k0, b_r);
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1 && lane == 0 && leader) {
    // ------------------------------- MMA issuer (leader CTA only) --------------------------------
    constexpr uint32_t idesc = make_idesc_bf16(BLOCK_M, BLOCK_N, A_MN, B_MN);
    constexpr uint64_t a_hi = A_MN ? make_smem_desc_hi(CHUNK_BYTES, 1024) : make_smem_desc_hi(16, 1024);
    constexpr uint64_t b_hi = B_MN ? make_smem_desc_hi(CHUNK_BYTES, 1024) : make_smem_desc_hi(16, 1024);
    constexpr uint32_t a_kstep = A_MN ? 2048u : 32u;
    constexpr uint32_t b_kstep = B_MN ? 2048u : 32u;
    int stage = 0;
    uint32_t phase = 0;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
      if (*abort_ptr != 0 || !mbar_wait_bounded(tempty_bar(acc_stage), acc_phase ^ 1u)) {
        raise_abort(LEANFFN_DEV_TIMEOUT_MMA);
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc_stage * BLOCK_N;
      for (int kb = 0; kb < kb_total; ++kb) {
        if (*abort_ptr != 0 || !mbar_wait_bounded(full_bar(stage), phase)) {
          raise_abort(LEANFFN_DEV_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint32_t sb = sa + A_BYTES;
#pragma unroll
        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
          const uint64_t da = make_smem_desc(sa + k * a_kstep, a_hi);
          const uint64_t db = make_smem_desc(sb + k * b_kstep, b_hi);
          umma_bf16_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit_pair(empty_bar(stage), 3u);  // frees this stage in both CTAs
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      umma_commit_pair(tfull_bar(acc_stage), 3u);  // accumulator complete, both CTAs' epilogues may read
      if (++acc_stage == 2) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  } else if (warp >= 2) {
    // ------------------------------- epilogue (both CTAs, own 128 rows) ---------------------------
    const EpiParams& ep = p.ep;
    const int quarter = warp & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t leader_tempty0 = map_to_cta(tempty_bar(0), 0);
    float* patch = reinterpret_cast<float*>(smem_gen + STAGES_ALLOC * STAGE_BYTES + 256) + (warp - 2) * EPI_PATCH_FLOATS;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs) {
      int m_blk, n_blk;
      tile_coords(tile, m_blk, n_blk);
      if (*abort_ptr != 0 || !mbar_wait_bounded(tfull_bar(acc_stage), acc_phase)) {
        if (lane == 0) raise_abort(LEANFFN_DEV_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const int64_t row0 = static_cast<int64_t>(m_blk) * BLOCK_M + rank * 128 + quarter * 32;
      const uint32_t t_acc = tmem_base + lane_addr + acc_stage * BLOCK_N;
      epilogue_tile<BLOCK_N>(ep, p.glu_split, t_acc, row0, n_blk, true, patch, lane, (warp - 2) >> 2, 2);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty0 + 8u * acc_stage);
      if (++acc_stage == 2) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ------------------------------- teardown ------------------------------------------------------
  __syncwarp();
  if (*abort_ptr != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the peer may still read this CTA's shared memory / arrive on its barriers until here
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// ---- host side -------------------------------------------------------------------------------------
bool make_tmap_bf16(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, uint32_t box_cols,
                    uint32_t box_rows, bool fp32 = false);

template <bool A_MN, bool B_MN>
static cudaError_t pair_launch_t(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& a2,
                                 const CUtensorMap& b2, const TcParams& p, cudaStream_t st) {
  auto kern = gemm_tcgen05_pair_kernel<A_MN, B_MN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(pair::THREADS, 1, 1);
  cfg.dynamicSmemBytes = pair::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // A persistent grid must be co-resident.  Clusters of two need both SMs in one GPC, so fewer pairs than
  // SMs / 2 may fit at a time (GPCs with an odd number of usable SMs): ask the runtime once per device.
  static int max_pairs[64] = {0};
  if (dev >= 0 && dev < 64 && max_pairs[dev] == 0) {
    int n = 0;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * (sm_count() / 2)), 1, 1);
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = sm_count() / 2;
    max_pairs[dev] = n;
    if (getenv("LEANFFN_DEBUG") != nullptr) fprintf(stderr, "leanffn: %d CTA pairs fit on device %d (%d SMs)\n", n, dev, sm_count());
  }
  int pairs = (dev >= 0 && dev < 64) ? max_pairs[dev] : sm_count() / 2;
  if (pairs > sm_count() / 2) pairs = sm_count() / 2;
  if (p.max_ctas > 0 && pairs > p.max_ctas / 2) pairs = p.max_ctas / 2;
  if (pairs > tiles) pairs = tiles;
  if (pairs < 1) pairs = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
  return cudaLaunchKernelEx(&cfg, kern, a, b, a2, b2, p);
}

// Dense products only (no block-sparse tables).  p.num_m_blocks / num_n_blocks count 256 x 256 tiles.
int32_t gemm_tcgen05_pair(bool a_mn, bool b_mn, const TcOperand& A, const TcOperand& B, const TcOperand* A2,
                          const TcOperand* B2, TcParams p, cudaStream_t st) {
  CUtensorMap ta, tb, ta2, tb2;
  auto encode = [&](CUtensorMap* m, const TcOperand& o, bool mn) {
    return make_tmap_bf16(m, o.ptr, o.rows, o.cols, o.ld, 64, mn ? 64 : 128);
  };
  if (!encode(&ta, A, a_mn) || !encode(&tb, B, b_mn)) return LEANFFN_ERR_DRIVER;
  if (A2 != nullptr && B2 != nullptr) {
    if (!encode(&ta2, *A2, a_mn) || !encode(&tb2, *B2, b_mn)) return LEANFFN_ERR_DRIVER;
  } else {
    ta2 = ta;
    tb2 = tb;
  }
  cudaError_t e;
  if (!a_mn && !b_mn) e = pair_launch_t<false, false>(ta, tb, ta2, tb2, p, st);
  else if (!a_mn && b_mn) e = pair_launch_t<false, true>(ta, tb, ta2, tb2, p, st);
  else if (a_mn && b_mn) e = pair_launch_t<true, true>(ta, tb, ta2, tb2, p, st);
  else return LEANFFN_ERR_UNSUPPORTED;
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}

}  // namespace leanffn
