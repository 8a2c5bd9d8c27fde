// Attention core on tcgen05: softmax(scale * Q.K^T + mask) . V per (batch, head) without the [q_len, kv_len]
// matrices ever reaching global memory, forward and backward.
//
// A CTA owns a 128-row tile; row r of every accumulator is TMEM lane r, and the threads that share a row split its
// columns (two per row in the forward pass, four in the backward pass).  All tiles are [128 rows x 64 columns] bf16
// boxes (16 KiB, 128-byte swizzle) fetched through a 4D tensor map over the [batch, len, heads, head_dim] view, so
// the head split and transposes of the reference are address arithmetic; head_dim > 64 takes two boxes.  The same
// bytes serve as the K-major operand of one product and the MN-major operand of another (a [128 x 64] box is 128 rows
// of 128 bytes either way), so every tile is fetched once:
//   forward, per key tile j:   S = Q_i . K_j^T -> softmax rows online -> P (bf16, written by the threads in the
//                              swizzled K-major layout) -> O_j = P . V_j, accumulated in registers with the
//                              running-maximum correction; thread 0 issues the loads and products, two CTAs per SM
//                              (head_dim <= 64) overlap one another's phases;
//   backward, per query tile i (one CTA per key tile j):
//                              S = Q_i . K_j^T, dP = dO_i . V_j^T -> P = exp2(S - lse), dS = P * (dP - delta)
//                              -> dV += P^T . dO_i, dK += dS^T . Q_i (TMEM, whole loop), dQ_i = dS . K_j (added
//                              to an fp32 buffer by TMA reductions); a dedicated warp issues the loads and
//                              products, the hand-overs are mbarriers.
// Every mbarrier wait is bounded; a wait that runs out sets the status word, every role leaves its loop and TMEM is
// freed.  Warp-collective tensor-memory loads sit behind warp-uniform conditions only.
#include <cstdlib>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "../../include/leanffn_b200.h"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace leanffn {

bool make_tmap_bf16_heads(CUtensorMap* out, const void* base, int64_t batch, int64_t len, int64_t heads,
                          int64_t head_dim, int64_t ld, int box_rows = 128);
bool make_tmap_f32_heads(CUtensorMap* out, void* base, int64_t batch, int64_t len, int64_t heads, int64_t head_dim);

namespace attn {

constexpr int TILE = 128;               // query rows / keys per tile
constexpr uint32_t BOX_BYTES = 128 * 64 * 2;   // one [128 x 64] bf16 box
constexpr uint32_t PS_BYTES = 2 * BOX_BYTES;   // a [128 x 128] bf16 matrix written by the threads
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
  int32_t B, H, Sq, Skv, d;
  int32_t causal;
  float scale;
  uint32_t drop_threshold;  // 0: no dropout on the probabilities
  float inv_keep;           // 1 / (1 - p)
  uint64_t seed, elem_offset;
  const float* mask;
  int64_t mask_sb, mask_sh, mask_sq;
  bf16* out;
  int64_t ld_out;
  float* lse;
  const float* delta;
  float* dq_acc;
  bf16* dk;
  bf16* dv;
  int64_t ld_dk, ld_dv;
  int32_t* status;
  long long wait_limit;
};

__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* tmap, uint32_t bar, int32_t x,
                                            int32_t y, int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// Adds a [128 x 32] fp32 box in shared memory (128-byte swizzle) to global memory through the TMA unit: one
// instruction instead of a thousand vector reductions from the SM; the adds themselves happen in L2.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* tmap, uint32_t smem_src, int32_t x, int32_t y,
                                                  int32_t z, int32_t w) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_src), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// 2^x on the special-function unit (one instruction; results below 2^-126 flush to zero, which is what a
// probability that small rounds to in bf16 anyway)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of the 16-byte piece `piece` (0..15: 8 keys each) of row `row` inside a thread-written [128 x 128]
// bf16 matrix laid out as two [128 x 64] K-major boxes with the 128-byte swizzle the tensor cores expect.
__device__ __forceinline__ uint32_t ps_offset(int row, int piece) {
  const int box = piece >> 3, j = piece & 7;
  return static_cast<uint32_t>(box) * BOX_BYTES + static_cast<uint32_t>(row >> 3) * 1024u +
         static_cast<uint32_t>(row & 7) * 128u + static_cast<uint32_t>((j ^ (row & 7)) << 4);
}

// The values of one 32-key chunk of a score row in log2 units: acc * scale_log2 + mask * log2(e), -inf where the
// key does not exist or the causal rule forbids it.
__device__ __forceinline__ void score_chunk(const uint32_t (&acc)[32], float (&v)[32], float scale_log2,
                                            const float* mask_row, int k0, int kv_len, int k_limit) {
#pragma unroll
  for (int c = 0; c < 32; ++c) v[c] = __uint_as_float(acc[c]) * scale_log2;
  if (mask_row != nullptr) {
    if (k0 + 32 <= kv_len && (reinterpret_cast<uintptr_t>(mask_row + k0) & 15u) == 0) {
      const float4* m4 = reinterpret_cast<const float4*>(mask_row + k0);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 m = __ldg(m4 + c);
        v[4 * c + 0] = fmaf(m.x, LOG2E, v[4 * c + 0]);
        v[4 * c + 1] = fmaf(m.y, LOG2E, v[4 * c + 1]);
        v[4 * c + 2] = fmaf(m.z, LOG2E, v[4 * c + 2]);
        v[4 * c + 3] = fmaf(m.w, LOG2E, v[4 * c + 3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (k0 + c < kv_len) v[c] = fmaf(__ldg(mask_row + k0 + c), LOG2E, v[c]);
    }
  }
  if (k0 + 32 > k_limit) {
#pragma unroll
    for (int c = 0; c < 32; ++c)
      if (k0 + c >= k_limit) v[c] = -INFINITY;
  }
}

// Dropout factors of 32 consecutive probabilities starting at element index e0: f[x] = 1 / (1 - p) if kept, else 0.
// Not inlined: the counter-based generator needs many registers; f lives in local memory.  `aligned` must be uniform
// over the warp (it is a property of kv_len and the stream offset, not of the row): the callers execute warp-collective
// tensor-memory loads right after, so no lane may take a different path here.
__device__ __noinline__ void dropout_factors(float* f, uint64_t e0, bool aligned, uint64_t seed, uint32_t threshold,
                                             float inv_keep) {
  if (aligned) {  // e0 is a multiple of 4: eight whole Philox groups
#pragma unroll 1
    for (int g = 0; g < 8; ++g) {
      bool keep[4];
      dropout_keep4((e0 >> 2) + g, seed, threshold, keep);
#pragma unroll
      for (int i = 0; i < 4; ++i) f[4 * g + i] = keep[i] ? inv_keep : 0.f;
    }
  } else {  // kv_len or the offset not a multiple of 4: the groups of four straddle the chunks
#pragma unroll 1
    for (int x = 0; x < 32; ++x) f[x] = dropout_keep1(e0 + x, seed, threshold) ? inv_keep : 0.f;
  }
  __syncwarp();
}

struct Smem {
  uint32_t base;     // 1024-aligned shared address of the tile area
  uint8_t* gen;      // the same address as a generic pointer
};

__device__ __forceinline__ Smem align_smem(uint8_t* raw) {
  Smem s;
  const uint32_t a = smem_u32(raw);
  s.base = (a + 1023u) & ~1023u;
  s.gen = raw + (s.base - a);
  return s;
}

// ------------------------------------------------------------------------------------------------------------
// Forward.  grid = (query tiles, heads, batch), late (long) query tiles first.  A CTA takes one tile of 128 query rows
// and walks over the keys 64 at a time; 4 compute warps (one thread per query row, all 64 keys of the step) + an issuing
// warp + a loading warp.  DPAD = head_dim rounded up to 32; DROP = dropout on the probabilities (its own
// instantiation, so that the counter-based generator costs the plain kernels nothing).
//
// Why 64 keys: one step of a CTA is a chain of hand-overs (scores complete -> exponentials -> arrive -> issue -> commit)
// whose latencies a CTA cannot hide from itself; what hides them is more CTAs per SM, and a CTA of this shape holds
// little: 128 TMEM columns (64 S / P, 64 O) and 48 KB of shared memory (Q, 2 x K, 2 x V of 64 rows) for head_dim <= 64,
// FOUR CTAs per SM; 256 columns and 96 KB above, two CTAs per SM.
//
// The output row O stays in tensor memory for the whole loop: the products P . V accumulate there.  The reference
// maximum of a row only moves when a step's maximum exceeds it by more than 2^8 (then the row of O and the
// denominator are rescaled, a tensor-memory load / store); otherwise probabilities are taken against the old reference
// and may reach 2^8, which bf16 and the fp32 sums hold without loss.  P replaces the scores in tensor memory (two bf16
// per column) and is the A operand of P . V from there.  Steps where the rule is plain (inside the key range, below
// the causal diagonal, unmasked) take ONE pass: probabilities against the old reference with no search for the step's
// maximum; the sum of the row's 64 probabilities, which the denominator needs anyway, tells whether that was safe (at
// most 2^14: no score exceeded the reference by more than 14); if not, in any row of the warp, the warp redoes the step
// with the two-pass rule before anything was stored.
// Lane 0 of the issuing warp issues every product and lane 0 of the loading warp makes every TMA request (a request
// costs its thread a few hundred clocks and the tile takes a microsecond or two to arrive).  A commit covers
// everything issued before it, so "S of step t + 1 is complete" also tells the compute warps that P . V of step t is.
//
// Per step t:  compute: wait S_t -> P = exp2(S - m) over S -> 4 arrivals on bar_p
//              issuer:  wait bar_p -> P . V of step t into O -> S_{t+1}
//              loader:  wait S_t -> request K_{t+2}, V_{t+1}
// Hand-overs are mbarriers with bounded waits only.
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units
constexpr int KSTEP = 64;
constexpr int FWD_COMPUTE_WARPS = 4;
constexpr int FWD_THREADS = 32 * (FWD_COMPUTE_WARPS + 2);
constexpr uint32_t KV_BOX_BYTES = KSTEP * 128;  // 64 rows of 128 bytes

template <int DPAD, bool DROP>
__global__ void __launch_bounds__(FWD_THREADS, DPAD <= 64 ? 4 : 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const Params p) {
  constexpr uint32_t TMEM_COLS = DPAD <= 64 ? 128 : 256, COL_O = 64;
  constexpr uint32_t DC = DPAD <= 64 ? 1 : 2;  // 64-column boxes per tile
  constexpr uint32_t Q_BYTES = DC * BOX_BYTES, KV_BYTES = DC * KV_BOX_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const Smem sm = align_smem(smem_raw);
  const uint32_t sQ = sm.base, sK0 = sQ + Q_BYTES, sV0 = sK0 + 2 * KV_BYTES;
  const uint32_t bar0 = sV0 + 2 * KV_BYTES;
  const uint32_t bar_q = bar0, bar_k0 = bar0 + 8 /* 2 */, bar_v0 = bar0 + 24 /* 2 */, bar_s = bar0 + 40;
  const uint32_t bar_o = bar0 + 48, bar_p = bar0 + 56, tmem_slot = bar0 + 64;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(sm.gen + Q_BYTES + 4 * KV_BYTES + 64);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = tid & 127;
  const bool issuer = warp == FWD_COMPUTE_WARPS, loader = warp == FWD_COMPUTE_WARPS + 1;
  const int nq = (p.Sq + TILE - 1) / TILE, nkv_all = (p.Skv + KSTEP - 1) / KSTEP;
  const int qt = nq - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int off = p.Skv - p.Sq;
  int steps = nkv_all;
  if (p.causal) {
    const int last_q = min(qt * TILE + TILE - 1, p.Sq - 1);
    const int last_k = last_q + off;  // largest key any row of the tile may see
    steps = last_k < 0 ? 0 : min(nkv_all, last_k / KSTEP + 1);
  }
  const long long limit = p.wait_limit > 0 ? p.wait_limit : WAIT_LIMIT_CYCLES;

  if (tid == 0) {
    for (int i = 0; i < 8; ++i) mbar_init(bar0 + 8 * i, i == 7 ? FWD_COMPUTE_WARPS : 1);
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t t_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);  // this warp's 32 lanes
  const uint32_t t_out = t_row + COL_O;
  bool ok = true;

  if (issuer) {
    if (lane == 0 && steps > 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, KSTEP, false, false);
      const uint32_t idesc_o = make_idesc_bf16(128, p.d, false, true);
      constexpr uint64_t k_major_hi = make_smem_desc_hi(16, 1024);
      constexpr uint64_t mn_major_hi = make_smem_desc_hi(KV_BOX_BYTES, 1024);
      auto issue_s = [&](int t) {  // S_t = Q . K_t^T: 64 columns, one product per 16 columns of the head
        const uint32_t sK = sK0 + (t & 1) * KV_BYTES;
        const int ksteps = p.d >> 4;
#pragma unroll
        for (int ks = 0; ks < 4 * static_cast<int>(DC); ++ks) {
          if (ks < ksteps)
            umma_bf16(tmem, make_smem_desc(sQ + (ks >> 2) * BOX_BYTES + (ks & 3) * 32u, k_major_hi),
                      make_smem_desc(sK + (ks >> 2) * KV_BOX_BYTES + (ks & 3) * 32u, k_major_hi), idesc_s,
                      ks > 0 ? 1u : 0u);
        }
        umma_commit(bar_s);
      };
      bool go = mbar_wait_bounded(bar_q, 0, limit) && mbar_wait_bounded(bar_k0, 0, limit);
      if (go) {
        tc_fence_after();
        issue_s(0);
      }
      for (int t = 0; t < steps && go; ++t) {
        go = mbar_wait_bounded(bar_p, t & 1, limit);  // P_t is in tensor memory, S_t has been read, O rescaled
        if (go) go = mbar_wait_bounded(bar_v0 + 8 * (t & 1), (t >> 1) & 1, limit);
        if (!go) break;
        tc_fence_after();
        const uint32_t sV = sV0 + (t & 1) * KV_BYTES;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)  // O += P . V_t over the 64 keys
          umma_bf16_tmem_a(tmem + COL_O, tmem + ks * 8, make_smem_desc(sV + ks * 2048u, mn_major_hi), idesc_o,
                           (t > 0 || ks > 0) ? 1u : 0u);
        if (t + 1 < steps) {
          go = mbar_wait_bounded(bar_k0 + 8 * ((t + 1) & 1), ((t + 1) >> 1) & 1, limit);  // requested a step ago
          if (!go) break;
          issue_s(t + 1);  // executes behind the products above, which read P_t from the columns it overwrites
        } else {
          umma_commit(bar_o);  // the last product: the output rows are complete
        }
      }
      if (!go && p.status != nullptr) atomicCAS(p.status, 0, LEANFFN_DEV_TIMEOUT_MMA);
    }
    __syncwarp();
  } else if (loader) {
    if (lane == 0 && steps > 0) {
      auto load_kv = [&](const CUtensorMap* m, uint32_t dst, uint32_t bar, int t) {
        mbar_arrive_expect_tx(bar, KV_BYTES);
        for (uint32_t c = 0; c < DC; ++c) tma_load_4d(dst + c * KV_BOX_BYTES, m, bar, c * 64, h, t * KSTEP, b);
      };
      mbar_arrive_expect_tx(bar_q, Q_BYTES);
      for (uint32_t c = 0; c < DC; ++c) tma_load_4d(sQ + c * BOX_BYTES, &tmQ, bar_q, c * 64, h, qt * TILE, b);
      load_kv(&tmK, sK0, bar_k0, 0);
      load_kv(&tmV, sV0, bar_v0, 0);
      if (steps > 1) load_kv(&tmK, sK0 + KV_BYTES, bar_k0 + 8, 1);
      bool go = true;
      for (int t = 0; t + 1 < steps && go; ++t) {
        // S_t complete: K_t is free; a commit covers everything issued before it, so P.V of step t - 1 is complete
        // too and the other V buffer is free.  (This thread cannot fall two steps behind: S_{t+2} needs the K
        // requested here.)
        go = mbar_wait_bounded(bar_s, t & 1, limit);
        if (!go) break;
        if (t + 2 < steps) load_kv(&tmK, sK0 + (t & 1) * KV_BYTES, bar_k0 + 8 * (t & 1), t + 2);
        load_kv(&tmV, sV0 + ((t + 1) & 1) * KV_BYTES, bar_v0 + 8 * ((t + 1) & 1), t + 1);
      }
      if (!go && p.status != nullptr) atomicCAS(p.status, 0, LEANFFN_DEV_TIMEOUT_PRODUCER);
    }
    __syncwarp();
  } else {
    const float scale_log2 = p.scale * LOG2E;
    const bool drop_aligned = ((p.Skv | static_cast<int>(p.elem_offset)) & 3) == 0;  // uniform: every chunk starts a Philox group
    auto wait_warp = [&](uint32_t bar, uint32_t parity) {  // the whole warp continues or the whole warp leaves
      return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, limit)) != 0;
    };
    const int q_row = qt * TILE + row;
    const int q_clamped = min(q_row, p.Sq - 1);
    const float* mask_row = p.mask == nullptr ? nullptr
                                              : p.mask + b * p.mask_sb + h * p.mask_sh + q_clamped * p.mask_sq;
    const int k_limit_row = p.causal ? min(p.Skv, q_row + off + 1) : p.Skv;
    const uint64_t drop_row = p.elem_offset + ((static_cast<uint64_t>(b) * p.H + h) * p.Sq + q_clamped) * p.Skv;
    float m_run = -INFINITY, l_run = 0.f;
    for (int t = 0; t < steps; ++t) {
      // S_t complete; a commit covers everything issued before it, so P.V of step t - 1 is complete too
      ok = wait_warp(bar_s, t & 1);
      if (!ok) break;
      tc_fence_after();
      const int k0 = t * KSTEP;
      // whole step inside the key range, below the causal diagonal for every row and unmasked: no per-element rule
      const bool plain = p.mask == nullptr && k0 + KSTEP <= p.Skv && scale_log2 > 0.f &&
                         (!p.causal || k0 + KSTEP - 1 <= qt * TILE + off);
      float row_sum = 0.f;
      // one pass against the OLD reference maximum where the rule is plain, checked by the row sum
      bool fast = DROP ? false : (plain && t > 0 && __all_sync(0xffffffffu, m_run > -INFINITY) != 0);
      if (fast) {
        uint32_t packed[2][16];
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t acc[32];
          tmem_ld_32x32(t_row + c * 32, acc);
          tmem_ld_wait();
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(acc[x]), scale_log2, -m_run));
            const float e1 = fast_exp2(fmaf(__uint_as_float(acc[x + 1]), scale_log2, -m_run));
            part[(x >> 1) & 3] += e0 + e1;
            packed[c][x >> 1] = pack_bf16x2(e0, e1);
          }
        }
        const float sum = (part[0] + part[1]) + (part[2] + part[3]);
        fast = __all_sync(0xffffffffu, sum <= 16384.f) != 0;
        if (fast) {
          tmem_st_32x16(t_row, packed[0]);
          tmem_st_32x16(t_row + 16, packed[1]);
          row_sum = sum;
        }
      }
      if (!fast) {
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t acc[32];
          tmem_ld_32x32(t_row + c * 32, acc);
          tmem_ld_wait();
          if (plain) {
#pragma unroll
            for (int x = 0; x < 32; ++x) mx = fmaxf(mx, __uint_as_float(acc[x]));
          } else {
            float v[32];
            score_chunk(acc, v, scale_log2, mask_row, k0 + c * 32, p.Skv, k_limit_row);
#pragma unroll
            for (int x = 0; x < 32; ++x) mx = fmaxf(mx, v[x]);
          }
        }
        if (plain) mx *= scale_log2;  // the scale is positive: the maximum commutes with it
        const bool move = mx > m_run + RESCALE_THRESHOLD || (m_run == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, move)) {
          const float m_new = move ? mx : m_run;
          const float alpha = (move && m_run > -INFINITY) ? fast_exp2(m_run - m_new) : 1.f;
          if (t > 0) {  // rows of O that exist already (uniform)
#pragma unroll
            for (int c = 0; c < DPAD / 32; ++c) {
              uint32_t acc[32];
              tmem_ld_32x32(t_out + c * 32, acc);
              tmem_ld_wait();
#pragma unroll
              for (int x = 0; x < 32; ++x) acc[x] = __float_as_uint(__uint_as_float(acc[x]) * alpha);
              tmem_st_32x32(t_out + c * 32, acc);
            }
            tmem_st_wait();
          }
          l_run *= alpha;
          m_run = m_new;
        }
        const float m_use = m_run == -INFINITY ? 0.f : m_run;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t acc[32];
          float v[32];
          tmem_ld_32x32(t_row + c * 32, acc);
          tmem_ld_wait();
          if (plain) {
#pragma unroll
            for (int x = 0; x < 32; ++x) v[x] = fast_exp2(fmaf(__uint_as_float(acc[x]), scale_log2, -m_use));
          } else {
            score_chunk(acc, v, scale_log2, mask_row, k0 + c * 32, p.Skv, k_limit_row);
#pragma unroll
            for (int x = 0; x < 32; ++x) v[x] = fast_exp2(v[x] - m_use);
          }
#pragma unroll
          for (int x = 0; x < 32; ++x) row_sum += v[x];
          if constexpr (DROP) {  // the denominator sums all probabilities, P . V only the kept ones
            float f[32];
            dropout_factors(f, drop_row + static_cast<uint64_t>(k0 + c * 32), drop_aligned, p.seed, p.drop_threshold, p.inv_keep);
#pragma unroll
            for (int x = 0; x < 32; ++x) v[x] *= f[x];
          }
          uint32_t packed[16];
#pragma unroll
          for (int x = 0; x < 16; ++x) packed[x] = pack_bf16x2(v[2 * x], v[2 * x + 1]);
          tmem_st_32x16(t_row + c * 16, packed);
        }
      }
      l_run += row_sum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
    }
    if (ok && steps > 0) ok = wait_warp(bar_o, 0);  // the last P.V
    if (!ok && lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, LEANFFN_DEV_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* dst = p.out + (static_cast<int64_t>(b) * p.Sq + q_row) * p.ld_out + static_cast<int64_t>(h) * p.d;
#pragma unroll
      for (int c = 0; c < DPAD / 16; ++c) {
        uint32_t o[16];
        if (steps > 0) {  // uniform
          tmem_ld_32x16(t_out + c * 16, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int x = 0; x < 16; ++x) o[x] = 0u;
        }
        if (q_row < p.Sq && c * 16 < p.d) {
          uint4 w[2];
          uint32_t* wp = reinterpret_cast<uint32_t*>(w);
#pragma unroll
          for (int x = 0; x < 8; ++x)
            wp[x] = pack_bf16x2(__uint_as_float(o[2 * x]) * inv, __uint_as_float(o[2 * x + 1]) * inv);
          *reinterpret_cast<uint4*>(dst + c * 16) = w[0];
          *reinterpret_cast<uint4*>(dst + c * 16 + 8) = w[1];
        }
      }
      // rows that saw no key at all get +inf so that the backward pass turns their probabilities into zeros
      if (q_row < p.Sq)
        p.lse[(static_cast<int64_t>(b) * p.H + h) * p.Sq + q_row] = l_run > 0.f ? m_run + log2f(l_run) : INFINITY;
    }
  }

  if (__syncthreads_and(ok) == 0) {  // a wait ran out: leave time for what is in flight before tensor memory goes back
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------------------
// delta[b, h, q] = sum_x dO[b, q, h, x] * O[b, q, h, x]
__global__ void attention_delta_kernel(const bf16* __restrict__ d_out, int64_t ld_dout, const bf16* __restrict__ out,
                                       int64_t ld_out, float* __restrict__ delta, int B, int H, int Sq, int d) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(B) * Sq * H;
  if (idx >= total) return;
  const int h = static_cast<int>(idx % H);
  const int64_t bq = idx / H;  // b * Sq + q
  const uint4* a = reinterpret_cast<const uint4*>(d_out + bq * ld_dout + static_cast<int64_t>(h) * d);
  const uint4* o = reinterpret_cast<const uint4*>(out + bq * ld_out + static_cast<int64_t>(h) * d);
  float s = 0.f;
  for (int x = 0; x < d / 8; ++x) {
    const uint4 av = __ldg(a + x), ov = __ldg(o + x);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
    const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 af = __bfloat1622float2(a2[i]), of = __bfloat1622float2(o2[i]);
      s = fmaf(af.x, of.x, s);
      s = fmaf(af.y, of.y, s);
    }
  }
  const int64_t b = bq / Sq, q = bq - b * Sq;
  delta[(b * H + h) * Sq + q] = s;
}

// ------------------------------------------------------------------------------------------------------------
// Backward.  grid = (key tiles, heads, batch).  16 compute warps + an issuing warp + a copy warp.
//
// Compute warps: four threads per row, thread group c = warp / 4 owns the 32 columns [32c, 32c + 32) of every
// 128-column accumulator row (no reduction across the threads of a row is needed: the row statistics lse and delta are
// inputs).  Lane 0 of the issuing warp issues every product; issuing blocks while the tensor cores' queue is full, so
// this thread does nothing else.  Lane 0 of the copy warp makes every TMA request (K, V once; Q / dO per tile as soon
// as a buffer is free; the reductions of the staged dQ tiles): a request costs its thread a few hundred clocks.
//
// Per query tile i:  group A(i) = {S = Q_i . K^T, dP = dO_i . V^T}          -> bar_a
//                    elementwise(i): P = exp2(S - lse), dS = P * (dP - delta) -> shared memory, 16 arrivals on bar_pds
//                    group B(i) = {dQ_i = dS . K -> bar_dq;  dV += P^T . dO_i, dK += dS^T . Q_i -> bar_b}
//                    read-out(i): dQ_i * scale added to the fp32 gradient in global memory -> 16 arrivals on bar_drain
// The only hand-overs are mbarriers with bounded waits: no block-wide barrier inside the loop.
// head_dim <= 64 (PIPE): three Q / dO buffers fetched three tiles ahead.  The compute warps say so (bar_sread) as soon
// as S_i and dP_i are in their registers, and A(i + 1) is issued right then: they never wait for scores.  dS goes to
// tensor memory first (two bf16 per column, bar_dst) and is the A operand of dQ_i from there, so that product runs
// while P and dS are copied to shared memory for dV / dK (the copies wait for bar_b of the tile before: the old P / dS
// are operands until then).  dQ has its own TMEM columns and is handed to the TMA unit through shared memory
// ([128 x 32] fp32 boxes, cp.reduce.async.bulk.tensor .add; bar_stage: boxes written, bar_sfree: boxes read).
// Order on the tensor cores: A(i + 1), dQ(i), dV/dK(i), A(i + 2), ...
// head_dim > 64: one Q / dO buffer; dS from shared memory; dQ_i reuses the S columns, so A(i + 1) waits for the
// read-out (bar_drain).
// Shared memory: K, V, NBUF x (Q, dO) (DC boxes each), P, dS (2 boxes each), PIPE: dQ staging (DPAD / 32 boxes).
// TMEM (512 columns): [0, 128) S; [128, 256) dP; PIPE: [256, 320) dV, [320, 384) dK, [384, 448) dQ, [448, 512) dS;
//                     otherwise [256, 384) dV, [384, 512) dK, dQ in [0, 128).
constexpr int BWD_COMPUTE_WARPS = 16;
constexpr int BWD_THREADS = 32 * (BWD_COMPUTE_WARPS + 2);  // + the issuing warp and the copy warp

template <int DPAD, bool DROP>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmdQ, const Params p) {
  constexpr bool PIPE = DPAD <= 64;
  constexpr int NBUF = PIPE ? 3 : 1;
  constexpr uint32_t COL_DV = 256, COL_DK = PIPE ? 320 : 384, COL_DQ = PIPE ? 384 : 0;
  constexpr uint32_t COL_DS = 448;  // PIPE only: dS as the tensor-memory A operand of dQ (two bf16 per column)
  extern __shared__ uint8_t smem_raw[];
  const Smem sm = align_smem(smem_raw);
  const int DC = (p.d + 63) >> 6;
  const uint32_t tile_bytes = DC * BOX_BYTES;
  const uint32_t sK = sm.base, sV = sK + tile_bytes, sQ0 = sV + tile_bytes;  // then per buffer: Q, dO
  const uint32_t sP = sQ0 + 2 * NBUF * tile_bytes, sdS = sP + PS_BYTES;
  const uint32_t bar0 = sdS + PS_BYTES;
  const uint32_t bar_kv = bar0, bar_a = bar0 + 8, bar_b = bar0 + 16, bar_dq = bar0 + 24, bar_pds = bar0 + 32;
  const uint32_t bar_drain = bar0 + 40, bar_q0 = bar0 + 96 /* NBUF barriers */, bar_stage = bar0 + 64, tmem_slot = bar0 + 72;
  const uint32_t bar_dst = bar0 + 80;  // PIPE only: dS is in tensor memory
  const uint32_t bar_sfree = bar0 + 88;  // PIPE only: the TMA unit has read the staging boxes
  const uint32_t bar_sread = bar0 + 48;  // PIPE only: S and dP of this tile are in registers
  uint8_t* gP = sm.gen + (2 + 2 * NBUF) * tile_bytes;
  uint8_t* gdS = gP + PS_BYTES;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gdS + PS_BYTES + 72);
  uint8_t* g_stage = gdS + PS_BYTES + 1024;  // PIPE only: DPAD / 32 boxes [128 x 32] fp32, 1024-byte aligned
  const uint32_t s_stage = sdS + PS_BYTES + 1024;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = warp >> 2, row = tid & 127;
  const bool issuer = warp == BWD_COMPUTE_WARPS, copier = warp == BWD_COMPUTE_WARPS + 1;
  const int nq = (p.Sq + TILE - 1) / TILE;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int off = p.Skv - p.Sq;
  int i_start = 0;
  if (p.causal) {
    const int first_q = kt * TILE - off;  // smallest query row that may see the first key of this tile
    i_start = first_q <= 0 ? 0 : first_q / TILE;
  }
  const int n_iter = max(nq - i_start, 0);
  const long long limit = p.wait_limit > 0 ? p.wait_limit : WAIT_LIMIT_CYCLES;

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(bar_a, 1);
    mbar_init(bar_b, 1);
    mbar_init(bar_dq, 1);
    mbar_init(bar_pds, BWD_COMPUTE_WARPS);
    mbar_init(bar_drain, BWD_COMPUTE_WARPS);
    mbar_init(bar_stage, BWD_COMPUTE_WARPS);
    mbar_init(bar_dst, BWD_COMPUTE_WARPS);
    mbar_init(bar_sfree, 1);
    mbar_init(bar_sread, BWD_COMPUTE_WARPS);
    for (int n = 0; n < NBUF; ++n) mbar_init(bar_q0 + 8 * n, 1);
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmdO);
    if (PIPE) prefetch_tmap(&tmdQ);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t t_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  bool ok = true;

  if (issuer) {
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);   // S and dP: both operands K-major
      const uint32_t idesc_t = make_idesc_bf16(128, p.d, true, true);     // dV, dK: P^T / dS^T (MN-major A), MN-major B
      const uint32_t idesc_q = make_idesc_bf16(128, p.d, false, true);    // dQ: dS K-major, K_j MN-major
      constexpr uint64_t k_major_hi = make_smem_desc_hi(16, 1024);
      constexpr uint64_t mn_major_hi = make_smem_desc_hi(BOX_BYTES, 1024);
      auto issue_a = [&](int buf) {
        const uint32_t sQ = sQ0 + 2 * buf * tile_bytes, sdO = sQ + tile_bytes;
        const int ksteps = p.d >> 4;
        for (int ks = 0; ks < ksteps; ++ks) {
          const uint32_t o = static_cast<uint32_t>(ks >> 2) * BOX_BYTES + static_cast<uint32_t>(ks & 3) * 32u;
          umma_bf16(tmem, make_smem_desc(sQ + o, k_major_hi), make_smem_desc(sK + o, k_major_hi), idesc_s, ks > 0 ? 1u : 0u);
          umma_bf16(tmem + 128, make_smem_desc(sdO + o, k_major_hi), make_smem_desc(sV + o, k_major_hi), idesc_s,
                    ks > 0 ? 1u : 0u);
        }
        umma_commit(bar_a);
      };
      auto issue_dq = [&]() {  // dQ[q, x] = sum_key dS[q, key] * K[key, x]: first, the compute warps wait for it
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          if constexpr (PIPE) {  // dS from tensor memory: the product does not wait for the copy in shared memory
            umma_bf16_tmem_a(tmem + COL_DQ, tmem + COL_DS + ks * 8, make_smem_desc(sK + ks * 2048u, mn_major_hi),
                             idesc_q, ks > 0 ? 1u : 0u);
          } else {
            const uint32_t oa = static_cast<uint32_t>(ks >> 2) * BOX_BYTES + static_cast<uint32_t>(ks & 3) * 32u;
            umma_bf16(tmem + COL_DQ, make_smem_desc(sdS + oa, k_major_hi), make_smem_desc(sK + ks * 2048u, mn_major_hi),
                      idesc_q, ks > 0 ? 1u : 0u);
          }
        }
        umma_commit(bar_dq);
      };
      auto issue_dv_dk = [&](int buf, uint32_t accumulate) {
        const uint32_t sQ = sQ0 + 2 * buf * tile_bytes, sdO = sQ + tile_bytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // dV[key, x] += sum_q P[q, key] * dO[q, x]
          umma_bf16(tmem + COL_DV, make_smem_desc(sP + ks * 2048u, mn_major_hi),
                    make_smem_desc(sdO + ks * 2048u, mn_major_hi), idesc_t, ks > 0 ? 1u : accumulate);
          // dK[key, x] += sum_q dS[q, key] * Q[q, x]
          umma_bf16(tmem + COL_DK, make_smem_desc(sdS + ks * 2048u, mn_major_hi),
                    make_smem_desc(sQ + ks * 2048u, mn_major_hi), idesc_t, ks > 0 ? 1u : accumulate);
        }
        umma_commit(bar_b);
      };

      bool go = mbar_wait_bounded(bar_kv, 0, limit) && mbar_wait_bounded(bar_q0, 0, limit);
      if (go) {
        tc_fence_after();
        issue_a(0);
      }
      for (int n = 0; n < n_iter && go; ++n) {
        const int buf = PIPE ? n % NBUF : 0;
        if (PIPE && n + 1 < n_iter) {
          // the next tile's scores go first: as soon as the compute warps hold S_i and dP_i in registers the columns
          // are free, and Q / dO of tile i + 1 were requested three tiles ago.  The compute warps then never wait
          // for scores: S_{i+1}, dP_{i+1} complete while they work on tile i.
          const int nb = (n + 1) % NBUF;
          go = mbar_wait_bounded(bar_sread, n & 1, limit) &&
               mbar_wait_bounded(bar_q0 + 8 * nb, ((n + 1) / NBUF) & 1, limit);
          if (!go) break;
          tc_fence_after();
          issue_a(nb);
        }
        // PIPE: dS is in tensor memory (dQ of the tile before drained); otherwise: P, dS written to shared memory
        go = mbar_wait_bounded(PIPE ? bar_dst : bar_pds, n & 1, limit);
        // PIPE: the staging boxes of the tile before have been read (dQ_i will be written there)
        if (PIPE && go && n > 0) go = mbar_wait_bounded(bar_sfree, (n - 1) & 1, limit);
        if (!go) break;
        tc_fence_after();
        issue_dq();
        if (PIPE) {
          // the compute warps keep the new P and dS in registers until bar_b says the old ones are no longer operands
          go = mbar_wait_bounded(bar_pds, n & 1, limit);  // P, dS are in shared memory too
          if (!go) break;
          tc_fence_after();
        }
        issue_dv_dk(buf, n == 0 ? 0u : 1u);
        if (!PIPE && n + 1 < n_iter) {
          // dQ_i lives in the S columns: the next scores wait until the compute warps have drained it
          go = mbar_wait_bounded(bar_drain, n & 1, limit) && mbar_wait_bounded(bar_q0, (n + 1) & 1, limit);
          if (!go) break;
          tc_fence_after();
          issue_a(0);
        }
      }
      if (!go && p.status != nullptr) atomicCAS(p.status, 0, LEANFFN_DEV_TIMEOUT_MMA);
    }
    __syncwarp();
  } else if (copier) {
    // Lane 0 does every TMA request: the loads (K, V once; Q / dO per tile as soon as their buffer is free) and, PIPE,
    // the reductions of the staged dQ tiles.  A request costs the requesting thread a few hundred clocks, which
    // neither the issuing thread nor a compute warp has to spare.
    if (lane == 0 && n_iter > 0) {
      auto load_boxes = [&](const CUtensorMap* m, uint32_t dst, uint32_t bar, int row0) {
        for (int c = 0; c < DC; ++c) tma_load_4d(dst + c * BOX_BYTES, m, bar, c * 64, h, row0, b);
      };
      auto load_q_do = [&](int i, int buf) {
        const uint32_t bar = bar_q0 + 8 * buf, dst = sQ0 + 2 * buf * tile_bytes;
        mbar_arrive_expect_tx(bar, 2 * tile_bytes);
        load_boxes(&tmQ, dst, bar, i * TILE);
        load_boxes(&tmdO, dst + tile_bytes, bar, i * TILE);
      };
      mbar_arrive_expect_tx(bar_kv, 2 * tile_bytes);
      load_boxes(&tmK, sK, bar_kv, kt * TILE);
      load_boxes(&tmV, sV, bar_kv, kt * TILE);
      load_q_do(i_start, 0);
      if (PIPE && n_iter > 1) load_q_do(i_start + 1, 1);
      if (PIPE && n_iter > 2) load_q_do(i_start + 2, 2);
      bool go = true;
      for (int n = 0; n < n_iter && go; ++n) {
        const int i = i_start + n;
        if (PIPE) {
          go = mbar_wait_bounded(bar_stage, n & 1, limit);  // all 16 warps have written their rows of dQ_i
          if (!go) break;
          for (int c = 0; c * 32 < p.d; ++c) tma_reduce_add_4d(&tmdQ, s_stage + c * BOX_BYTES, c * 32, h, i * TILE, b);
          bulk_commit_group();
          bulk_wait_group_read0();
          mbar_arrive(bar_sfree);  // dQ_{i+1} may be issued: its read-out writes the boxes again
        }
        // dV / dK of tile i complete (and with them everything issued before): Q_i, dO_i are free.  (This thread
        // cannot fall two tiles behind: those products of a later tile need the Q / dO requested here.)
        const int next = PIPE ? n + NBUF : n + 1;
        if (next < n_iter) {
          go = mbar_wait_bounded(bar_b, n & 1, limit);
          if (!go) break;
          load_q_do(i_start + next, PIPE ? n % NBUF : 0);
        }
      }
      if (PIPE) bulk_wait_group0();  // the reductions of this block have been performed
      if (!go && p.status != nullptr) atomicCAS(p.status, 0, LEANFFN_DEV_TIMEOUT_PRODUCER);
    }
    __syncwarp();
  } else {
    const float scale_log2 = p.scale * LOG2E;
    const int k0 = kt * TILE;
    auto wait_warp = [&](uint32_t bar, uint32_t parity) {  // the whole warp continues or the whole warp leaves
      return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, limit)) != 0;
    };
    for (int n = 0; n < n_iter; ++n) {
      const int i = i_start + n;
      // row statistics of this tile: requested before the wait for the scores
      const int q_row = i * TILE + row;
      const bool q_valid = q_row < p.Sq;
      const int q_clamped = min(q_row, p.Sq - 1);
      const int64_t stat = (static_cast<int64_t>(b) * p.H + h) * p.Sq + q_clamped;
      const float lse = q_valid ? __ldg(p.lse + stat) : INFINITY;  // +inf: the row's probabilities become zero
      const float dlt = q_valid ? __ldg(p.delta + stat) : 0.f;
      const float* mask_row = p.mask == nullptr ? nullptr
                                                : p.mask + b * p.mask_sb + h * p.mask_sh + q_clamped * p.mask_sq;
      const int k_limit_row = p.causal ? min(p.Skv, q_row + off + 1) : p.Skv;

      ok = wait_warp(bar_a, n & 1);
      if (!ok) break;
      tc_fence_after();
      {
        const int c = chunk;
        uint32_t acc[32], dp[32];
        float v[32];
        tmem_ld_32x32(t_row + c * 32, acc);
        tmem_ld_32x32(t_row + 128 + c * 32, dp);
        tmem_ld_wait();
        if constexpr (PIPE) {  // the score columns are free for the next tile
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_sread);
        }
        // whole tile inside the key range, below the causal diagonal for every row and unmasked: no per-element rule
        const bool plain = p.mask == nullptr && k0 + TILE <= p.Skv && (!p.causal || k0 + TILE - 1 <= i * TILE + off);
        if (plain) {
#pragma unroll
          for (int x = 0; x < 32; ++x) v[x] = fast_exp2(fmaf(__uint_as_float(acc[x]), scale_log2, -lse));
        } else {
          score_chunk(acc, v, scale_log2, mask_row, k0 + c * 32, p.Skv, k_limit_row);
#pragma unroll
          for (int x = 0; x < 32; ++x) v[x] = fast_exp2(v[x] - lse);
        }
        uint4 wp[4];        // this thread's 32 probabilities, packed bf16
        uint32_t wd[16];    // and its 32 score gradients
        if constexpr (DROP) {
          // dV takes the kept probabilities scaled by 1 / (1 - p); the gradient of a dropped probability is zero
          float f[32];
          const uint64_t e0 = p.elem_offset + ((static_cast<uint64_t>(b) * p.H + h) * p.Sq + q_clamped) * p.Skv +
                              static_cast<uint64_t>(k0 + c * 32);
          dropout_factors(f, e0, ((p.Skv | static_cast<int>(p.elem_offset)) & 3) == 0, p.seed, p.drop_threshold, p.inv_keep);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            wp[q4].x = pack_bf16x2(v[8 * q4 + 0] * f[8 * q4 + 0], v[8 * q4 + 1] * f[8 * q4 + 1]);
            wp[q4].y = pack_bf16x2(v[8 * q4 + 2] * f[8 * q4 + 2], v[8 * q4 + 3] * f[8 * q4 + 3]);
            wp[q4].z = pack_bf16x2(v[8 * q4 + 4] * f[8 * q4 + 4], v[8 * q4 + 5] * f[8 * q4 + 5]);
            wp[q4].w = pack_bf16x2(v[8 * q4 + 6] * f[8 * q4 + 6], v[8 * q4 + 7] * f[8 * q4 + 7]);
          }
#pragma unroll
          for (int x = 0; x < 32; ++x) dp[x] = __float_as_uint(__uint_as_float(dp[x]) * f[x]);
        } else {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            wp[q4].x = pack_bf16x2(v[8 * q4 + 0], v[8 * q4 + 1]);
            wp[q4].y = pack_bf16x2(v[8 * q4 + 2], v[8 * q4 + 3]);
            wp[q4].z = pack_bf16x2(v[8 * q4 + 4], v[8 * q4 + 5]);
            wp[q4].w = pack_bf16x2(v[8 * q4 + 6], v[8 * q4 + 7]);
          }
        }
#pragma unroll
        for (int x = 0; x < 32; ++x) v[x] *= __uint_as_float(dp[x]) - dlt;  // dS; the score scale is applied to dQ / dK
#pragma unroll
        for (int x = 0; x < 16; ++x) wd[x] = pack_bf16x2(v[2 * x], v[2 * x + 1]);
        if constexpr (PIPE) {
          // dS into tensor memory as the A operand of dQ_i = dS . K: that product starts now, not after the copies below
          tmem_st_32x16(t_row + COL_DS + c * 16, wd);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_dst);
        }
        // P and dS of the tile before are operands of its dV / dK products until bar_b completes
        if (n > 0) ok = wait_warp(bar_b, (n - 1) & 1);
        if (ok) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint32_t o = ps_offset(row, c * 4 + q4);
            *reinterpret_cast<uint4*>(gP + o) = wp[q4];
            *reinterpret_cast<uint4*>(gdS + o) = make_uint4(wd[4 * q4], wd[4 * q4 + 1], wd[4 * q4 + 2], wd[4 * q4 + 3]);
          }
        }
      }
      if (!ok) break;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pds);

      ok = wait_warp(bar_dq, n & 1);
      if (!ok) break;
      tc_fence_after();
      if (PIPE) {
        // dQ_i * scale goes to shared memory as [128 x 32] fp32 boxes (swizzled like every other tile) and from there
        // to the fp32 gradient in global memory by TMA reductions: rows beyond q_len and columns beyond head_dim are
        // clipped by the tensor map
        if (chunk < DPAD / 32) {  // uniform per warp
          uint32_t acc[32];
          tmem_ld_32x32(t_row + COL_DQ + chunk * 32, acc);
          tmem_ld_wait();
#pragma unroll
          for (int x = 0; x < 8; ++x)
            *reinterpret_cast<float4*>(g_stage + ps_offset(row, chunk * 8 + x)) =
                make_float4(__uint_as_float(acc[4 * x]) * p.scale, __uint_as_float(acc[4 * x + 1]) * p.scale,
                            __uint_as_float(acc[4 * x + 2]) * p.scale, __uint_as_float(acc[4 * x + 3]) * p.scale);
          fence_proxy_async_smem();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_stage);  // the copy warp hands the staged tile to the TMA unit
      } else {
        float* dst = p.dq_acc + (static_cast<int64_t>(b) * p.Sq + q_clamped) * (static_cast<int64_t>(p.H) * p.d) +
                     static_cast<int64_t>(h) * p.d;
        if (chunk < DPAD / 32) {  // uniform per warp
          const int c = chunk;
          uint32_t acc[32];
          tmem_ld_32x32(t_row + COL_DQ + c * 32, acc);
          tmem_ld_wait();
          if (q_valid) {
#pragma unroll
            for (int x = 0; x < 32; x += 4)
              if (c * 32 + x < p.d)
                red_add_v4(dst + c * 32 + x, __uint_as_float(acc[x]) * p.scale, __uint_as_float(acc[x + 1]) * p.scale,
                           __uint_as_float(acc[x + 2]) * p.scale, __uint_as_float(acc[x + 3]) * p.scale);
          }
        }
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_drain);
    }
    if (ok && n_iter > 0) ok = wait_warp(bar_b, (n_iter - 1) & 1);  // the last dV / dK products
    if (ok) {
      tc_fence_after();
      // tcgen05.ld is warp-collective: every thread reads its lane, only the rows that exist are stored
      const int key = kt * TILE + row;
      const bool key_valid = key < p.Skv;
      const int64_t key_row = static_cast<int64_t>(b) * p.Skv + min(key, p.Skv - 1);
      bf16* dv = p.dv + key_row * p.ld_dv + static_cast<int64_t>(h) * p.d;
      bf16* dk = p.dk + key_row * p.ld_dk + static_cast<int64_t>(h) * p.d;
      if (chunk < DPAD / 32) {  // uniform per warp
        const int c = chunk;
        uint32_t av[32], ak[32];
        if (n_iter > 0) {
          tmem_ld_32x32(t_row + COL_DV + c * 32, av);
          tmem_ld_32x32(t_row + COL_DK + c * 32, ak);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) av[x] = 0u, ak[x] = 0u;
        }
        if (key_valid) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            if (c * 32 + x < p.d) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(av[x + 0]), __uint_as_float(av[x + 1]));
              w.y = pack_bf16x2(__uint_as_float(av[x + 2]), __uint_as_float(av[x + 3]));
              w.z = pack_bf16x2(__uint_as_float(av[x + 4]), __uint_as_float(av[x + 5]));
              w.w = pack_bf16x2(__uint_as_float(av[x + 6]), __uint_as_float(av[x + 7]));
              *reinterpret_cast<uint4*>(dv + c * 32 + x) = w;
              w.x = pack_bf16x2(__uint_as_float(ak[x + 0]) * p.scale, __uint_as_float(ak[x + 1]) * p.scale);
              w.y = pack_bf16x2(__uint_as_float(ak[x + 2]) * p.scale, __uint_as_float(ak[x + 3]) * p.scale);
              w.z = pack_bf16x2(__uint_as_float(ak[x + 4]) * p.scale, __uint_as_float(ak[x + 5]) * p.scale);
              w.w = pack_bf16x2(__uint_as_float(ak[x + 6]) * p.scale, __uint_as_float(ak[x + 7]) * p.scale);
              *reinterpret_cast<uint4*>(dk + c * 32 + x) = w;
            }
          }
        }
      }
    } else if (lane == 0 && p.status != nullptr) {
      atomicCAS(p.status, 0, LEANFFN_DEV_TIMEOUT_EPILOGUE);
    }
  }
  // teardown: after a timeout give copies and products still in flight time to land before the memory is released
  if (!__syncthreads_and(ok)) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------------------
// Rotary embedding (and plain conversion) over [batch * len, heads, head_dim]; one thread per pair (x_left, x_right).
template <typename TI, typename TO>
__global__ void rotary_kernel(const TI* __restrict__ x, int64_t ld_x, const float* __restrict__ cos_t,
                              const float* __restrict__ sin_t, int64_t ld_t, TO* __restrict__ y, int64_t ld_y,
                              int64_t rows, int len, int heads, int d, int inverse) {
  const int half = d >> 1;
  const int64_t per_row = static_cast<int64_t>(heads) * half;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const int64_t row = idx / per_row;
  const int rem = static_cast<int>(idx - row * per_row);
  const int hh = rem / half, i = rem - hh * half;
  const int pos = static_cast<int>(row % len);
  const int64_t xo = row * ld_x + static_cast<int64_t>(hh) * d, yo = row * ld_y + static_cast<int64_t>(hh) * d;
  const float xl = static_cast<float>(x[xo + i]), xr = static_cast<float>(x[xo + half + i]);
  float yl = xl, yr = xr;
  if (cos_t != nullptr) {
    const float cl = cos_t[pos * ld_t + i], cr = cos_t[pos * ld_t + half + i];
    const float sl = sin_t[pos * ld_t + i], sr = sin_t[pos * ld_t + half + i];
    if (!inverse) {
      yl = xl * cl - xr * sl;   // x * cos + (-x_right) * sin
      yr = xr * cr + xl * sr;   // x * cos + x_left * sin
    } else {
      yl = xl * cl + xr * sr;
      yr = xr * cr - xl * sl;
    }
  }
  y[yo + i] = static_cast<TO>(yl);
  y[yo + half + i] = static_cast<TO>(yr);
}

// Same, eight pairs per thread with 16-byte (bf16) / 32-byte (fp32) accesses: half = head_dim / 2 a multiple of 8.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h2[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  uint4 w;
  w.x = pack_bf16x2(v[0], v[1]);
  w.y = pack_bf16x2(v[2], v[3]);
  w.z = pack_bf16x2(v[4], v[5]);
  w.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = w;
}

template <typename TI, typename TO>
__global__ void rotary_vec_kernel(const TI* __restrict__ x, int64_t ld_x, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, int64_t ld_t, TO* __restrict__ y, int64_t ld_y,
                                  int64_t rows, int len, int heads, int d, int inverse) {
  const int half = d >> 1, vecs = half >> 3;
  const int64_t per_row = static_cast<int64_t>(heads) * vecs;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const int64_t row = idx / per_row;
  const int rem = static_cast<int>(idx - row * per_row);
  const int hh = rem / vecs, i = (rem - hh * vecs) * 8;
  const int pos = static_cast<int>(row % len);
  const int64_t xo = row * ld_x + static_cast<int64_t>(hh) * d + i, yo = row * ld_y + static_cast<int64_t>(hh) * d + i;
  float xl[8], xr[8], yl[8], yr[8];
  load8(x + xo, xl);
  load8(x + xo + half, xr);
  if (cos_t != nullptr) {
    float cl[8], cr[8], sl[8], sr[8];
    load8(cos_t + pos * ld_t + i, cl);
    load8(cos_t + pos * ld_t + half + i, cr);
    load8(sin_t + pos * ld_t + i, sl);
    load8(sin_t + pos * ld_t + half + i, sr);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (!inverse) {
        yl[k] = xl[k] * cl[k] - xr[k] * sl[k];
        yr[k] = xr[k] * cr[k] + xl[k] * sr[k];
      } else {
        yl[k] = xl[k] * cl[k] + xr[k] * sr[k];
        yr[k] = xr[k] * cr[k] - xl[k] * sl[k];
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) yl[k] = xl[k], yr[k] = xr[k];
  }
  store8(y + yo, yl);
  store8(y + yo + half, yr);
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int32_t validate(const leanffn_attention_desc* d, bool backward) {
  if (d == nullptr || d->q == nullptr || d->k == nullptr || d->v == nullptr || d->out == nullptr || d->lse == nullptr)
    return LEANFFN_ERR_NULL;
  if (d->batch <= 0 || d->heads <= 0 || d->q_len <= 0 || d->kv_len <= 0) return LEANFFN_ERR_SHAPE;
  if (d->head_dim < 16 || d->head_dim > 128 || d->head_dim % 16 != 0) return LEANFFN_ERR_UNSUPPORTED;
  const int64_t width = static_cast<int64_t>(d->heads) * d->head_dim;
  if (d->ld_q < width || d->ld_k < width || d->ld_v < width || d->ld_out < width) return LEANFFN_ERR_SHAPE;
  if (d->ld_q % 8 || d->ld_k % 8 || d->ld_v % 8 || d->ld_out % 8) return LEANFFN_ERR_ALIGN;
  if (!aligned16(d->q) || !aligned16(d->k) || !aligned16(d->v) || !aligned16(d->out)) return LEANFFN_ERR_ALIGN;
  if (d->batch > 65535 || d->heads > 65535) return LEANFFN_ERR_TOO_LARGE;
  if (!(d->dropout_p >= 0.f) || d->dropout_p >= 1.f) return LEANFFN_ERR_SHAPE;
  if (backward) {
    if (d->d_out == nullptr || d->delta == nullptr || d->dq_accum == nullptr || d->dk == nullptr || d->dv == nullptr)
      return LEANFFN_ERR_NULL;
    if (d->ld_dout < width || d->ld_dk < width || d->ld_dv < width) return LEANFFN_ERR_SHAPE;
    if (d->ld_dout % 8 || d->ld_dk % 8 || d->ld_dv % 8) return LEANFFN_ERR_ALIGN;
    if (!aligned16(d->d_out) || !aligned16(d->dk) || !aligned16(d->dv) || !aligned16(d->dq_accum)) return LEANFFN_ERR_ALIGN;
  }
  return LEANFFN_OK;
}

static Params make_params(const leanffn_attention_desc* d) {
  Params p{};
  p.B = d->batch, p.H = d->heads, p.Sq = d->q_len, p.Skv = d->kv_len, p.d = d->head_dim;
  p.causal = d->causal;
  p.scale = d->scale;
  p.drop_threshold = d->dropout_p > 0.f ? dropout_threshold(d->dropout_p) : 0u;
  p.inv_keep = d->dropout_p > 0.f ? 1.f / (1.f - d->dropout_p) : 1.f;
  p.seed = d->seed, p.elem_offset = d->elem_offset;
  p.mask = d->mask;
  p.mask_sb = d->mask_stride_b, p.mask_sh = d->mask_stride_h, p.mask_sq = d->mask_stride_q;
  p.out = static_cast<bf16*>(d->out);
  p.ld_out = d->ld_out;
  p.lse = d->lse;
  p.delta = d->delta;
  p.dq_acc = d->dq_accum;
  p.dk = static_cast<bf16*>(d->dk);
  p.dv = static_cast<bf16*>(d->dv);
  p.ld_dk = d->ld_dk, p.ld_dv = d->ld_dv;
  p.status = d->status_word;
  p.wait_limit = d->wait_limit_cycles;
  return p;
}

template <typename K>
static cudaError_t set_smem(K kern, size_t bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
}

}  // namespace attn
}  // namespace leanffn

using namespace leanffn;

extern "C" int32_t leanffn_attention_forward(const leanffn_attention_desc* d, void* stream) {
  const int32_t v = attn::validate(d, false);
  if (v != LEANFFN_OK) return v;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap tq, tk, tv;
  if (!make_tmap_bf16_heads(&tq, d->q, d->batch, d->q_len, d->heads, d->head_dim, d->ld_q) ||
      !make_tmap_bf16_heads(&tk, d->k, d->batch, d->kv_len, d->heads, d->head_dim, d->ld_k, attn::KSTEP) ||
      !make_tmap_bf16_heads(&tv, d->v, d->batch, d->kv_len, d->heads, d->head_dim, d->ld_v, attn::KSTEP))
    return LEANFFN_ERR_DRIVER;
  const attn::Params p = attn::make_params(d);
  cudaError_t e;
  const int dc = (d->head_dim + 63) / 64;
  const size_t smem = dc * (attn::BOX_BYTES + 4 * attn::KV_BOX_BYTES) + 128 + 1024;
  const dim3 grid((d->q_len + attn::TILE - 1) / attn::TILE, d->heads, d->batch);
#define ATTN_FWD(DPAD)                                                             \
  {                                                                                \
    auto kern = p.drop_threshold != 0u ? attn::attention_fwd_kernel<DPAD, true>    \
                                       : attn::attention_fwd_kernel<DPAD, false>;  \
    e = attn::set_smem(kern, smem);                                                \
    if (e == cudaSuccess) {                                                        \
      kern<<<grid, attn::FWD_THREADS, smem, st>>>(tq, tk, tv, p);                  \
      e = cudaGetLastError();                                                      \
    }                                                                              \
  }
  if (d->head_dim <= 32) ATTN_FWD(32)
  else if (d->head_dim <= 64) ATTN_FWD(64)
  else if (d->head_dim <= 96) ATTN_FWD(96)
  else ATTN_FWD(128)
#undef ATTN_FWD
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}

extern "C" int32_t leanffn_attention_backward(const leanffn_attention_desc* d, void* stream) {
  const int32_t v = attn::validate(d, true);
  if (v != LEANFFN_OK) return v;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap tq, tk, tv, tdo;
  if (!make_tmap_bf16_heads(&tq, d->q, d->batch, d->q_len, d->heads, d->head_dim, d->ld_q) ||
      !make_tmap_bf16_heads(&tk, d->k, d->batch, d->kv_len, d->heads, d->head_dim, d->ld_k) ||
      !make_tmap_bf16_heads(&tv, d->v, d->batch, d->kv_len, d->heads, d->head_dim, d->ld_v) ||
      !make_tmap_bf16_heads(&tdo, d->d_out, d->batch, d->q_len, d->heads, d->head_dim, d->ld_dout))
    return LEANFFN_ERR_DRIVER;
  const attn::Params p = attn::make_params(d);
  const int64_t rows = static_cast<int64_t>(d->batch) * d->q_len * d->heads;
  cudaError_t e = cudaMemsetAsync(d->dq_accum, 0, static_cast<size_t>(rows) * d->head_dim * sizeof(float), st);
  if (e != cudaSuccess) return 1000 + static_cast<int32_t>(e);
  attn::attention_delta_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, st>>>(
      static_cast<const bf16*>(d->d_out), d->ld_dout, static_cast<const bf16*>(d->out), d->ld_out, d->delta, d->batch,
      d->heads, d->q_len, d->head_dim);
  e = cudaGetLastError();
  if (e != cudaSuccess) return 1000 + static_cast<int32_t>(e);
  const int dc = (d->head_dim + 63) / 64;
  // head_dim <= 64: three Q / dO buffers and the dQ staging boxes ([128 x 32] fp32 each)
  const int dpad = (d->head_dim + 31) / 32 * 32;
  const size_t smem = (dc == 1 ? 8 : 4) * dc * attn::BOX_BYTES + 2 * attn::PS_BYTES + 1024 + 1024 +
                      (dc == 1 ? (dpad / 32) * attn::BOX_BYTES : 0);
  CUtensorMap tdq;
  if (!make_tmap_f32_heads(&tdq, d->dq_accum, d->batch, d->q_len, d->heads, d->head_dim)) return LEANFFN_ERR_DRIVER;
  const dim3 grid((d->kv_len + attn::TILE - 1) / attn::TILE, d->heads, d->batch);
#define ATTN_BWD(DPAD)                                                             \
  {                                                                                \
    auto kern = p.drop_threshold != 0u ? attn::attention_bwd_kernel<DPAD, true>    \
                                       : attn::attention_bwd_kernel<DPAD, false>;  \
    e = attn::set_smem(kern, smem);                                                \
    if (e == cudaSuccess) {                                                        \
      kern<<<grid, attn::BWD_THREADS, smem, st>>>(tq, tk, tv, tdo, tdq, p);                 \
      e = cudaGetLastError();                                                      \
    }                                                                              \
  }
  if (d->head_dim <= 32) ATTN_BWD(32)
  else if (d->head_dim <= 64) ATTN_BWD(64)
  else if (d->head_dim <= 96) ATTN_BWD(96)
  else ATTN_BWD(128)
#undef ATTN_BWD
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}

extern "C" int32_t leanffn_rotary(const void* x, int32_t x_dtype, int64_t ld_x, const float* cos_table,
                                  const float* sin_table, int64_t ld_table, void* y, int32_t y_dtype, int64_t ld_y,
                                  int32_t batch, int32_t len, int32_t heads, int32_t head_dim, int32_t inverse,
                                  void* stream) {
  if (x == nullptr || y == nullptr) return LEANFFN_ERR_NULL;
  if ((cos_table == nullptr) != (sin_table == nullptr)) return LEANFFN_ERR_NULL;
  if (batch <= 0 || len <= 0 || heads <= 0 || head_dim <= 0 || head_dim % 2 != 0) return LEANFFN_ERR_SHAPE;
  const int64_t width = static_cast<int64_t>(heads) * head_dim;
  if (ld_x < width || ld_y < width || (cos_table != nullptr && ld_table < head_dim)) return LEANFFN_ERR_SHAPE;
  if ((x_dtype != LEANFFN_F32 && x_dtype != LEANFFN_BF16) || (y_dtype != LEANFFN_F32 && y_dtype != LEANFFN_BF16))
    return LEANFFN_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rows = static_cast<int64_t>(batch) * len;
  const int half = head_dim / 2;
  // eight pairs per thread where every access is a whole aligned vector; one pair per thread otherwise
  const auto vec_ok = [](const void* p, int64_t ld, int32_t dtype) {
    const int64_t bytes = dtype == LEANFFN_BF16 ? 2 : 4;
    return (reinterpret_cast<uintptr_t>(p) % 16 == 0) && (ld * bytes) % 16 == 0;
  };
  const bool vec = half % 8 == 0 && vec_ok(x, ld_x, x_dtype) && vec_ok(y, ld_y, y_dtype) &&
                   (cos_table == nullptr || (vec_ok(cos_table, ld_table, LEANFFN_F32) && vec_ok(sin_table, ld_table, LEANFFN_F32)));
  const int64_t total = rows * heads * (vec ? half / 8 : half);
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
#define ROTARY(TI, TO)                                                                                              \
  if (vec)                                                                                                          \
    attn::rotary_vec_kernel<TI, TO><<<blocks, 256, 0, st>>>(static_cast<const TI*>(x), ld_x, cos_table, sin_table,  \
                                                            ld_table, static_cast<TO*>(y), ld_y, rows, len, heads,  \
                                                            head_dim, inverse);                                     \
  else                                                                                                              \
    attn::rotary_kernel<TI, TO><<<blocks, 256, 0, st>>>(static_cast<const TI*>(x), ld_x, cos_table, sin_table,      \
                                                        ld_table, static_cast<TO*>(y), ld_y, rows, len, heads,      \
                                                        head_dim, inverse)
  if (x_dtype == LEANFFN_BF16 && y_dtype == LEANFFN_BF16) { ROTARY(bf16, bf16); }
  else if (x_dtype == LEANFFN_BF16) { ROTARY(bf16, float); }
  else if (y_dtype == LEANFFN_BF16) { ROTARY(float, bf16); }
  else { ROTARY(float, float); }
#undef ROTARY
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}
