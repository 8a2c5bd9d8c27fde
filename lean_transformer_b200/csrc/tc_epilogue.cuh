// Epilogue of the tcgen05 GEMM kernels.  A warp reads a 32-row x 32-column block of the fp32 accumulator from
// tensor memory (tcgen05.ld gives lane i the 32 columns of row i), adds the bias, rounds to bf16 and transposes the
// block through a private shared-memory patch so that four neighbouring lanes own 64 consecutive bytes of ONE
// output row; the fused epilogue then runs with fully used 32-byte sectors on every global load and store:
//   lane l, step i (0..3):  row = 8*i + l/4,  columns (l%4)*8 .. +7 of the block.
// The patch is exchanged as packed bf16 in 16-byte pieces (4 vector stores + 4 vector loads per lane and block):
// the main loop's TMA writes and tensor-core operand reads keep shared memory busy, so the epilogue has to be
// frugal with it.  Every intermediate of the fused block is a bf16 tensor in the unfused formulation, hence the
// early rounding changes no result.  Plain fp32 outputs (weight gradients into fp32 masters) keep an fp32 exchange.
// Shared by the one-CTA and the CTA-pair kernels; EPI_WARPS warps split the column blocks of a tile.
#pragma once
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace leanffn {

#ifndef LEANFFN_EPI_LOOKAHEAD
#define LEANFFN_EPI_LOOKAHEAD 0
#endif

// Measurement builds (-DLEANFFN_ABLATE_RUNTIME) can leave out phases of the fused epilogues at run time to see what
// each costs (results are then wrong on purpose); in product builds the mask is the constant 0 and folds away.
//   1: no residual / pre-activation loads   2: no global stores   4: no activation arithmetic   8: no column sums
//   16: no shared-memory transposition      32: no tensor-memory read
#ifdef LEANFFN_ABLATE_RUNTIME
#define LEANFFN_ABLATE_MASK(ep) ((ep).ablate)
#else
#define LEANFFN_ABLATE_MASK(ep) 0
#endif

constexpr int EPI_PATCH_FLOATS = 32 * 33;  // per-warp patch: fp32 exchange uses row pitch 33 (conflict-free);
                                           // the bf16 exchange uses its first 2 KiB

__device__ __forceinline__ void load8(const void* base, int32_t dtype, int64_t elem, float (&v)[8]) {
  if (dtype == LEANFFN_BF16) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(static_cast<const bf16*>(base) + elem));
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u[h]);
      v[2 * h] = __low2float(b);
      v[2 * h + 1] = __high2float(b);
    }
  } else {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem);
    const float4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  }
}
__device__ __forceinline__ void store8(void* base, int32_t dtype, int64_t elem, const float (&v)[8]) {
  if (dtype == LEANFFN_BF16) {
    uint4 w;
    w.x = pack_bf16x2(v[0], v[1]);
    w.y = pack_bf16x2(v[2], v[3]);
    w.z = pack_bf16x2(v[4], v[5]);
    w.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(static_cast<bf16*>(base) + elem) = w;
  } else {
    float4* p = reinterpret_cast<float4*>(static_cast<float*>(base) + elem);
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

__device__ __forceinline__ void unpack8(const uint4& w, float (&v)[8]) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u[h]);
    v[2 * h] = __low2float(b);
    v[2 * h + 1] = __high2float(b);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 w;
  w.x = pack_bf16x2(v[0], v[1]);
  w.y = pack_bf16x2(v[2], v[3]);
  w.z = pack_bf16x2(v[4], v[5]);
  w.w = pack_bf16x2(v[6], v[7]);
  return w;
}
// Product of two packed bf16 pairs, rounded to nearest even.  The exact product of two bf16 values fits an fp32
// mantissa, so this equals "multiply in fp32, round to bf16" bit for bit: one instruction for two elements and no
// unpacking, which matters because the fused epilogues are bound by instruction issue, not by memory.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint4 mul8(const uint4& a, const uint4& b) {
  return make_uint4(mul_bf16x2(a.x, b.x), mul_bf16x2(a.y, b.y), mul_bf16x2(a.z, b.z), mul_bf16x2(a.w, b.w));
}
// acc[0..7] += the 8 bf16 values packed in w
__device__ __forceinline__ void add_packed8(float* acc, const uint4& w) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    acc[2 * h] += __uint_as_float(u[h] << 16);
    acc[2 * h + 1] += __uint_as_float(u[h] & 0xFFFF0000u);
  }
}
#ifndef LEANFFN_EPI_STREAMING_STORES
#define LEANFFN_EPI_STREAMING_STORES 0
#endif
__device__ __forceinline__ void store_packed8(void* base, int32_t dtype, int64_t elem, const uint4& w) {
  if (dtype == LEANFFN_BF16) {
#if LEANFFN_EPI_STREAMING_STORES
    __stcs(reinterpret_cast<uint4*>(static_cast<bf16*>(base) + elem), w);  // written once, read by a later kernel
#else
    *reinterpret_cast<uint4*>(static_cast<bf16*>(base) + elem) = w;
#endif
  } else {
    float v[8];
    unpack8(w, v);
    store8(base, dtype, elem, v);
  }
}

// Atomic add (relaxed, system scope: the target may be another GPU's memory) of 8 consecutive elements.
__device__ __forceinline__ void red_add_packed8(void* base, int64_t elem, const uint4& w) {
  asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(static_cast<bf16*>(base) + elem),
               "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w)
               : "memory");
}
__device__ __forceinline__ void red_add_f32x8(void* base, int64_t elem, const float (&v)[8]) {
  float* p = static_cast<float*>(base) + elem;
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]),
               "f"(v[3])
               : "memory");
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + 4), "f"(v[4]), "f"(v[5]), "f"(v[6]),
               "f"(v[7])
               : "memory");
}
// Replica that owns `row` when the result is scattered over ranks (row blocks dealt round-robin).
__device__ __forceinline__ void* scatter_target(const EpiParams& ep, int64_t row) {
  const uint32_t owner = (static_cast<uint32_t>(row) >> ep.scatter_shift) % static_cast<uint32_t>(ep.scatter_world);
  return ep.scatter_D[owner];
}

// Bias of the 32 columns first .. first+31 (same for every lane: broadcast loads).  Columns at or beyond `limit`
// read as 0; limit and first are multiples of 8.
__device__ __forceinline__ void load_bias32(const void* bias, int32_t dtype, int64_t first, int64_t limit,
                                            float (&b)[32]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (bias != nullptr && first + 8 * c < limit) load8(bias, dtype, first + 8 * c, t);
#pragma unroll
    for (int q = 0; q < 8; ++q) b[8 * c + q] = t[q];
  }
}

// Byte offset of 16-byte piece `chunk` (8 bf16 columns) of `row` inside the bf16 patch.  Row pitch 64 B with the
// piece index XOR-ed by bits 1-2 of the row: both the row-wise vector stores (8 lanes = 8 rows, one piece) and the
// transposed vector loads (8 lanes = 2 rows x 4 pieces) touch 8 distinct 16-byte bank groups.
__device__ __forceinline__ uint32_t patch_offset(int row, int chunk) {
  return static_cast<uint32_t>(row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4));
}

// TMEM block (lane = row) + bias, rounded to bf16 ->  w[i] = 8 packed values of (row 8*i + lane/4,
// columns (lane%4)*8 .. +7) of the block.
__device__ __forceinline__ void load_block_bf16(uint32_t taddr, float* patch, int lane, bool valid,
                                                const float (&bias)[32], uint4 (&w)[4], bool has_bias = true,
                                                int ablate = 0) {
  uint32_t r[32];
  __syncwarp();
  if (ablate & 32) {
#pragma unroll
    for (int q = 0; q < 32; ++q) r[q] = 0x3f000000u + lane + q;
  } else {
    tmem_ld_32x32(taddr, r);
    tmem_ld_wait();
  }
  char* base = reinterpret_cast<char*>(patch);
  if (ablate & 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) f[q] = __uint_as_float(r[8 * i + q]);
      w[i] = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    }
    return;
  }
  if (!valid) {  // empty reduction (warp-uniform): the accumulator was never written
#pragma unroll
    for (int q = 0; q < 32; ++q) r[q] = 0u;
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float f[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) f[q] = __uint_as_float(r[8 * c + q]);
    if (has_bias) {  // warp-uniform
#pragma unroll
      for (int q = 0; q < 8; ++q) f[q] += bias[8 * c + q];
    }
    uint4 p;
    p.x = pack_bf16x2(f[0], f[1]);
    p.y = pack_bf16x2(f[2], f[3]);
    p.z = pack_bf16x2(f[4], f[5]);
    p.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(base + patch_offset(lane, c)) = p;
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = *reinterpret_cast<const uint4*>(base + patch_offset(8 * i + (lane >> 2), lane & 3));
  __syncwarp();
}

// TMEM block (lane = row) -> v[i][j] = element (row 8*i + lane/4, column (lane%4)*8 + j) of the block.
__device__ __forceinline__ void load_block_transposed(uint32_t taddr, float* patch, int lane, bool valid,
                                                      float (&v)[4][8]) {
  uint32_t r[32];
  __syncwarp();
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) patch[lane * 33 + j] = valid ? __uint_as_float(r[j]) : 0.f;
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) v[i][j] = patch[(8 * i + (lane >> 2)) * 33 + (lane & 3) * 8 + j];
  __syncwarp();
}

// Column sums over the 32 rows of a block.  Each lane holds, for its 8 columns ((lane % 4) * 8 .. + 7), the sum over its
// own 4 rows of NV / 8 tensors (NV = 8 or 16 values).  The 8 lanes that share a column group differ in lane bits 2-4;
// recursive halving over those bits (xor 16, 8, 4) leaves every lane with NV / 8 finished sums: value index
// ((lane >> 4) & 1) * NV/2 + ((lane >> 3) & 1) * NV/4 + ((lane >> 2) & 1) * NV/8 + j.  NV - NV/8 shuffles in total.
template <int NV>
__device__ __forceinline__ void halve_columns(float (&v)[NV], int lane, float (&out)[NV / 8]) {
  float a[NV / 2];
  {
    const bool hi = (lane & 16) != 0;
#pragma unroll
    for (int j = 0; j < NV / 2; ++j) {
      const float send = hi ? v[j] : v[j + NV / 2];
      const float keep = hi ? v[j + NV / 2] : v[j];
      a[j] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
  }
  float b[NV / 4];
  {
    const bool hi = (lane & 8) != 0;
#pragma unroll
    for (int j = 0; j < NV / 4; ++j) {
      const float send = hi ? a[j] : a[j + NV / 4];
      const float keep = hi ? a[j + NV / 4] : a[j];
      b[j] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
  }
  {
    const bool hi = (lane & 4) != 0;
#pragma unroll
    for (int j = 0; j < NV / 8; ++j) {
      const float send = hi ? b[j] : b[j + NV / 8];
      const float keep = hi ? b[j + NV / 8] : b[j];
      out[j] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
  }
}

// Which 32-column blocks of a tile a warp takes: the warps that share a lane quarter walk the blocks round-robin
// (share, share + shares, ...).  Giving each warp pairs of neighbouring blocks, so that both 64-byte halves of every
// 128-byte line are touched by one warp back to back, was measured and changes nothing.
__device__ __forceinline__ int epi_block(int j, int share, int shares) { return share + j * shares; }
__device__ __forceinline__ int epi_block_count(int num_blocks, int share, int shares) {
  return (num_blocks - share + shares - 1) / shares;
}

// Activation on 8 values.  ACT >= 0: one inlined activation.  ACT < 0: the run-time switch lives in ONE
// out-of-line copy, so rarely used activations do not bloat (and evict) the hot epilogue code.
static __device__ __noinline__ void act_fwd8_generic(int act, float* x) {
  for (int q = 0; q < 8; ++q) x[q] = act_fwd<true>(act, x[q]);
}
static __device__ __noinline__ void act_fwd_bwd8_generic(int act, float* x, float* d) {
  for (int q = 0; q < 8; ++q) {
    float y, dd;
    act_fwd_bwd<true>(act, x[q], y, dd);
    x[q] = y, d[q] = dd;
  }
}
template <int ACT>
__device__ __forceinline__ void act_fwd8(int act, const float (&x)[8], float (&y)[8]) {
  if constexpr (ACT >= 0) {
#pragma unroll
    for (int q = 0; q < 8; ++q) y[q] = act_fwd_t<ACT, true>(act, x[q]);
  } else {
#pragma unroll
    for (int q = 0; q < 8; ++q) y[q] = x[q];
    act_fwd8_generic(act, y);
  }
}
template <int ACT>
__device__ __forceinline__ void act_fwd_bwd8(int act, const float (&x)[8], float (&y)[8], float (&d)[8]) {
  if constexpr (ACT >= 0) {
#pragma unroll
    for (int q = 0; q < 8; ++q) act_fwd_bwd_t<ACT, true>(act, x[q], y[q], d[q]);
  } else {
#pragma unroll
    for (int q = 0; q < 8; ++q) y[q] = x[q];
    act_fwd_bwd8_generic(act, y, d);
  }
}

// One warp's share of a 128-row accumulator tile: TMEM lanes [quarter*32, +32), column blocks
// block_begin, block_begin + block_step, ...  t_acc = TMEM address of (lane quarter*32, first column of the tile);
// row0 = global row of TMEM lane quarter*32; n_blk = tile index along N (gated forward: along the
// intermediate dimension).  KIND / ACT are compile-time so that each launch runs a small, cache-resident loop.
template <int BLOCK_N, int KIND, int ACT>
__device__ __forceinline__ void epilogue_tile_t(const EpiParams& ep, int glu_split, uint32_t t_acc, int64_t row0,
                                                int n_blk, bool acc_valid, float* patch, int lane, int block_begin,
                                                int block_step) {
  const int sub_row = lane >> 2;        // + 8*i
  const int sub_col = (lane & 3) * 8;   // within the 32-column block
  if constexpr (KIND == LEANFFN_EPI_GLU_FWD) {
    if constexpr (BLOCK_N == 256) {
      // tile columns [0,128): gate, [128,256): linear half; output feature j = n_blk*128 + column
      const int inter = glu_split;
#pragma unroll 1
      for (int jb = 0; jb < epi_block_count(4, block_begin, block_step); ++jb) {
        const int blk = epi_block(jb, block_begin, block_step);
        const int64_t j0 = static_cast<int64_t>(n_blk) * 128 + blk * 32;
        const int64_t j = j0 + sub_col;
        const bool live = j < inter;
        uint4 g[4], l[4];
        {
          float bias[32];
          load_bias32(ep.bias, ep.bias_dtype, j0, inter, bias);
          load_block_bf16(t_acc + blk * 32, patch, lane, acc_valid, bias, g, ep.bias != nullptr);
        }
        {
          float bias[32];
          load_bias32(ep.bias, ep.bias_dtype, inter + j0, 2 * static_cast<int64_t>(inter), bias);
          load_block_bf16(t_acc + 128 + blk * 32, patch, lane, acc_valid, bias, l, ep.bias != nullptr);
        }
        if (!live) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int64_t row = row0 + 8 * i + sub_row;
          if (row >= ep.M) continue;
          store_packed8(ep.D, ep.d_dtype, row * ep.ldd + j, g[i]);
          store_packed8(ep.D, ep.d_dtype, row * ep.ldd + inter + j, l[i]);
          float gf[8], h[8];
          unpack8(g[i], gf);
          act_fwd8<ACT>(ep.act, gf, h);
          // hid = bf16(act(gate)) * lin, as packed bf16 products
          store_packed8(ep.D2, ep.d_dtype, row * ep.ldd2 + j, mul8(pack8(h), l[i]));
        }
      }
    }
    return;
  } else if constexpr (KIND == LEANFFN_EPI_STORE) {
    if (ep.d_dtype != LEANFFN_BF16) {
      // full-precision output: fp32 exchange
#pragma unroll 1
      for (int jb = 0; jb < epi_block_count(BLOCK_N / 32, block_begin, block_step); ++jb) {
        const int blk = epi_block(jb, block_begin, block_step);
        const int64_t col = static_cast<int64_t>(n_blk) * BLOCK_N + blk * 32 + sub_col;
        const bool live = col < ep.N;
        float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (live && ep.bias != nullptr) load8(ep.bias, ep.bias_dtype, col, b);
        float v[4][8];
        load_block_transposed(t_acc + blk * 32, patch, lane, acc_valid, v);
        if (!live) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int64_t row = row0 + 8 * i + sub_row;
          if (row >= ep.M) continue;
#pragma unroll
          for (int q = 0; q < 8; ++q) v[i][q] += b[q];
          if (ep.aux != nullptr && ep.aux_dtype == LEANFFN_F32) {
            // running sum over slices of a long reduction axis.  aux may be D itself, written earlier in THIS launch by
            // this very thread: read it through L2 (a non-coherent read-only load could return the stale value)
            float prev[8];
            {
              const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(ep.aux) + row * ep.ldaux + col);
              const float4 lo = __ldcg(src), hi = __ldcg(src + 1);
              prev[0] = lo.x, prev[1] = lo.y, prev[2] = lo.z, prev[3] = lo.w;
              prev[4] = hi.x, prev[5] = hi.y, prev[6] = hi.z, prev[7] = hi.w;
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) v[i][q] += prev[q];
          }
          if (ep.scatter_world > 0)
            red_add_f32x8(scatter_target(ep, row), row * ep.ldd + col, v[i]);
          else
            store8(ep.D, ep.d_dtype, row * ep.ldd + col, v[i]);
        }
      }
      return;
    }
#pragma unroll 1
    for (int jb = 0; jb < epi_block_count(BLOCK_N / 32, block_begin, block_step); ++jb) {
      const int blk = epi_block(jb, block_begin, block_step);
      const int64_t col0 = static_cast<int64_t>(n_blk) * BLOCK_N + blk * 32;
      const int64_t col = col0 + sub_col;
      const bool live = col < ep.N;
      uint4 w[4];
      {
        float bias[32];
        load_bias32(ep.bias, ep.bias_dtype, col0, ep.N, bias);
        load_block_bf16(t_acc + blk * 32, patch, lane, acc_valid, bias, w, ep.bias != nullptr);
      }
      if (!live) continue;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t row = row0 + 8 * i + sub_row;
        if (row >= ep.M) continue;
        if (ep.scatter_world > 0)
          red_add_packed8(scatter_target(ep, row), row * ep.ldd + col, w[i]);
        else
          store_packed8(ep.D, ep.d_dtype, row * ep.ldd + col, w[i]);
      }
    }
  } else {
    // The residual / pre-activation rows (bf16) of a block are requested before the block is read from tensor memory
    // and transposed, and stay packed in registers until used; the tile's rows were asked into L2 while the warp
    // waited for the accumulator (epilogue_prefetch_aux), so the request is an L2 hit that the transposition hides.
    // (Requesting one block further ahead costs 32 more registers per thread, which spilled in the hot loop.)
    constexpr bool LOOKAHEAD = LEANFFN_EPI_LOOKAHEAD != 0;
    const int ab = LEANFFN_ABLATE_MASK(ep);
    uint32_t sink = 0;  // measurement builds: keeps arithmetic alive when the stores are left out
    constexpr bool HAS_AUX =
        KIND == LEANFFN_EPI_DROPOUT_RESIDUAL || KIND == LEANFFN_EPI_GLU_BWD || KIND == LEANFFN_EPI_ACT_BWD;
    constexpr int NUM_BLOCKS = BLOCK_N / 32;
    uint4 n0[4], n1[4];
    auto request_aux = [&](int blk) {
      const int64_t col = static_cast<int64_t>(n_blk) * BLOCK_N + blk * 32 + sub_col;
      const bool live = col < ep.N && ep.aux != nullptr;
      const bf16* aux = static_cast<const bf16*>(ep.aux);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t row = row0 + 8 * i + sub_row;
        const bool ok = live && row < ep.M;
        n0[i] = n1[i] = make_uint4(0u, 0u, 0u, 0u);
        if (ab & 1) {
          n0[i] = n1[i] = make_uint4(0x3f003e80u, 0x3e003d80u, 0x3f003e80u, 0x3e003d80u);
        } else if (ok) {
          if (KIND == LEANFFN_EPI_DROPOUT_RESIDUAL && ep.aux_dtype == LEANFFN_F32) {
            // fp32 residual: the 8 columns fill both register sets (n0: columns 0-3, n1: columns 4-7)
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const float*>(ep.aux) + row * ep.ldaux + col);
            n0[i] = __ldg(src);
            n1[i] = __ldg(src + 1);
          } else {
            n0[i] = __ldg(reinterpret_cast<const uint4*>(aux + row * ep.ldaux + col));
            if constexpr (KIND == LEANFFN_EPI_GLU_BWD)
              n1[i] = __ldg(reinterpret_cast<const uint4*>(aux + row * ep.ldaux + ep.N + col));
          }
        }
      }
    };
    const int my_blocks = epi_block_count(NUM_BLOCKS, block_begin, block_step);
    if constexpr (HAS_AUX && LOOKAHEAD) {
      if (my_blocks > 0) request_aux(epi_block(0, block_begin, block_step));
    }
#pragma unroll 1
    for (int jb = 0; jb < my_blocks; ++jb) {
      const int blk = epi_block(jb, block_begin, block_step);
      const int64_t col0 = static_cast<int64_t>(n_blk) * BLOCK_N + blk * 32;
      const int64_t col = col0 + sub_col;
      const bool live = col < ep.N;
      uint4 c0[4], c1[4];
      if constexpr (HAS_AUX) {
        if constexpr (!LOOKAHEAD) request_aux(blk);
#pragma unroll
        for (int i = 0; i < 4; ++i) c0[i] = n0[i], c1[i] = n1[i];
        if constexpr (LOOKAHEAD) {
          if (jb + 1 < my_blocks) request_aux(epi_block(jb + 1, block_begin, block_step));
        }
      }
      uint4 w[4];
      {
        float bias[32];
        load_bias32(ep.bias, ep.bias_dtype, col0, ep.N, bias);
        load_block_bf16(t_acc + blk * 32, patch, lane, acc_valid, bias, w, ep.bias != nullptr, ab);
      }
      constexpr bool IS_BWD = KIND == LEANFFN_EPI_GLU_BWD || KIND == LEANFFN_EPI_ACT_BWD;
      constexpr int NCS = KIND == LEANFFN_EPI_GLU_BWD ? 16 : 8;
      float cs[NCS];  // backward kinds: this lane's column sums of the ROUNDED values it stores (bias gradient)
#pragma unroll
      for (int q = 0; q < NCS; ++q) cs[q] = 0.f;
      const bool want_cs = IS_BWD && ep.colsum != nullptr && !(ab & 8);  // warp-uniform
      if (!live && !want_cs) continue;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t row = row0 + 8 * i + sub_row;
        if (row >= ep.M || !live) continue;
        float x[8];
        unpack8(w[i], x);
        if constexpr (KIND == LEANFFN_EPI_ACT_FWD) {
          float h[8];
          act_fwd8<ACT>(ep.act, x, h);
          store_packed8(ep.D, ep.d_dtype, row * ep.ldd + col, w[i]);
          store8(ep.D2, ep.d_dtype, row * ep.ldd2 + col, h);
        } else if constexpr (KIND == LEANFFN_EPI_DROPOUT_RESIDUAL) {
          if (ep.threshold != 0u) {
            const uint64_t e0 = ep.elem_offset + static_cast<uint64_t>(row) * ep.N + col;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              bool keep[4];
              dropout_keep4((e0 >> 2) + q, ep.seed, ep.threshold, keep);
#pragma unroll
              for (int h = 0; h < 4; ++h) x[q * 4 + h] = keep[h] ? x[q * 4 + h] * ep.keep_scale : 0.f;
            }
          }
          float res[8];
          if (ep.aux_dtype == LEANFFN_F32) {
            res[0] = __uint_as_float(c0[i].x), res[1] = __uint_as_float(c0[i].y);
            res[2] = __uint_as_float(c0[i].z), res[3] = __uint_as_float(c0[i].w);
            res[4] = __uint_as_float(c1[i].x), res[5] = __uint_as_float(c1[i].y);
            res[6] = __uint_as_float(c1[i].z), res[7] = __uint_as_float(c1[i].w);
          } else {
            unpack8(c0[i], res);
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) x[q] += res[q];
          store8(ep.D, ep.d_dtype, row * ep.ldd + col, x);
        } else if constexpr (KIND == LEANFFN_EPI_GLU_BWD) {
          // w = dHid[row, col..] (packed); aux = pre [M, 2N] (c0 gate, c1 linear); D = dPre [M, 2N]; D2 = hid (optional).
          // The activation and its derivative are computed in fp32 from the gate, rounded once, and every product of
          // two bf16 tensors (as in the unfused formulation, where each is a bf16 tensor) is a packed bf16 product.
          float gate[8], y[8], d[8];
          unpack8(c0[i], gate);
          if (ab & 4) {
#pragma unroll
            for (int q = 0; q < 8; ++q) y[q] = gate[q], d[q] = 1.0f;
          } else {
            act_fwd_bwd8<ACT>(ep.act, gate, y, d);
          }
          const uint4 y2 = pack8(y), d2 = pack8(d);
          const uint4 dl = mul8(w[i], y2);                 // d/d(linear half) = dHid * act(gate)
          const uint4 dg = mul8(mul8(w[i], c1[i]), d2);    // d/d(gate) = dHid * lin * act'(gate)
          if (ab & 2) {
            const uint4 hv = mul8(y2, c1[i]);
            sink ^= dg.x ^ dg.y ^ dg.z ^ dg.w ^ dl.x ^ dl.y ^ dl.z ^ dl.w ^ hv.x ^ hv.y ^ hv.z ^ hv.w;
          } else {
            store_packed8(ep.D, ep.d_dtype, row * ep.ldd + col, dg);
            store_packed8(ep.D, ep.d_dtype, row * ep.ldd + ep.N + col, dl);
            if (ep.D2 != nullptr) store_packed8(ep.D2, ep.d_dtype, row * ep.ldd2 + col, mul8(y2, c1[i]));  // remat hid
          }
          if (want_cs) {
            add_packed8(cs, dg);
            add_packed8(cs + 8, dl);
          }
        } else if constexpr (KIND == LEANFFN_EPI_ACT_BWD) {
          float pre[8], y[8], d[8];
          unpack8(c0[i], pre);
          act_fwd_bwd8<ACT>(ep.act, pre, y, d);
          const uint4 dx = mul8(w[i], pack8(d));
          store_packed8(ep.D, ep.d_dtype, row * ep.ldd + col, dx);
          if (ep.D2 != nullptr) store8(ep.D2, ep.d_dtype, row * ep.ldd2 + col, y);
          if (want_cs) add_packed8(cs, dx);
        }
      }
      if constexpr (IS_BWD) {
        if (want_cs) {
          // every lane takes part in the exchange (dead lanes contribute zeros); row0 is a multiple of 32
          float fin[NCS / 8];
          halve_columns<NCS>(cs, lane, fin);
          if (row0 < ep.M) {
            float* prow = ep.colsum + (row0 >> 5) * ep.ldcolsum;
            if constexpr (KIND == LEANFFN_EPI_GLU_BWD) {
              // value index = half * 8 + column offset: half 0 = gate columns, half 1 = linear columns
              const int off = ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2;
              const int64_t c = ((lane & 16) ? ep.N : 0) + col + off;
              if (col + off < ep.N) *reinterpret_cast<float2*>(prow + c) = make_float2(fin[0], fin[1]);
            } else {
              const int off = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
              if (col + off < ep.N) prow[col + off] = fin[0];
            }
          }
        }
      }
    }
    if (sink == 0x9E3779B9u && ep.D != nullptr) *static_cast<uint32_t*>(ep.D) = sink;  // never true in practice
  }
}

// Ask L2 for the residual / pre-activation rows that epilogue_tile will read for the same arguments.  Called while
// the warp would otherwise sit waiting for the accumulator, so the epilogue's own loads find their data on chip.
// One lane per 64-byte row segment issues the request.
template <int BLOCK_N>
__device__ __forceinline__ void epilogue_prefetch_aux(const EpiParams& ep, int64_t row0, int n_blk, int lane,
                                                      int block_begin, int block_step) {
  const bool has_aux = ep.kind == LEANFFN_EPI_DROPOUT_RESIDUAL || ep.kind == LEANFFN_EPI_GLU_BWD ||
                       ep.kind == LEANFFN_EPI_ACT_BWD;
  if (!has_aux || ep.aux == nullptr || (lane & 3) != 0) return;
  const int esize = ep.aux_dtype == LEANFFN_BF16 ? 2 : 4;
  const char* aux = static_cast<const char*>(ep.aux);
#pragma unroll 1
  for (int jb = 0; jb < epi_block_count(BLOCK_N / 32, block_begin, block_step); ++jb) {
    const int blk = epi_block(jb, block_begin, block_step);
    const int64_t col = static_cast<int64_t>(n_blk) * BLOCK_N + blk * 32;
    if (col >= ep.N) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t row = row0 + 8 * i + (lane >> 2);
      if (row >= ep.M) continue;
      const char* p = aux + (row * ep.ldaux + col) * esize;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
      if (esize == 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + 64));
      if (ep.kind == LEANFFN_EPI_GLU_BWD) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + ep.N * esize));
    }
  }
}

template <int BLOCK_N, int KIND>
__device__ __forceinline__ void epilogue_tile_act(const EpiParams& ep, int glu_split, uint32_t t_acc, int64_t row0,
                                                  int n_blk, bool acc_valid, float* patch, int lane, int block_begin,
                                                  int block_step) {
  // gelu_fused and silu get their own inlined loops; everything else shares the out-of-line switch
  if (ep.act == LEANFFN_ACT_GELU_TANH)
    epilogue_tile_t<BLOCK_N, KIND, LEANFFN_ACT_GELU_TANH>(ep, glu_split, t_acc, row0, n_blk, acc_valid, patch, lane,
                                                          block_begin, block_step);
  else if (ep.act == LEANFFN_ACT_SILU)
    epilogue_tile_t<BLOCK_N, KIND, LEANFFN_ACT_SILU>(ep, glu_split, t_acc, row0, n_blk, acc_valid, patch, lane,
                                                     block_begin, block_step);
  else
    epilogue_tile_t<BLOCK_N, KIND, -1>(ep, glu_split, t_acc, row0, n_blk, acc_valid, patch, lane, block_begin,
                                       block_step);
}

template <int BLOCK_N>
__device__ __forceinline__ void epilogue_tile(const EpiParams& ep, int glu_split, uint32_t t_acc, int64_t row0,
                                              int n_blk, bool acc_valid, float* patch, int lane, int block_begin,
                                              int block_step) {
#define LEANFFN_EPI_ARGS ep, glu_split, t_acc, row0, n_blk, acc_valid, patch, lane, block_begin, block_step
  switch (ep.kind) {
    case LEANFFN_EPI_STORE: epilogue_tile_t<BLOCK_N, LEANFFN_EPI_STORE, -1>(LEANFFN_EPI_ARGS); break;
    case LEANFFN_EPI_DROPOUT_RESIDUAL: epilogue_tile_t<BLOCK_N, LEANFFN_EPI_DROPOUT_RESIDUAL, -1>(LEANFFN_EPI_ARGS); break;
    case LEANFFN_EPI_GLU_FWD: epilogue_tile_act<BLOCK_N, LEANFFN_EPI_GLU_FWD>(LEANFFN_EPI_ARGS); break;
    case LEANFFN_EPI_ACT_FWD: epilogue_tile_act<BLOCK_N, LEANFFN_EPI_ACT_FWD>(LEANFFN_EPI_ARGS); break;
    case LEANFFN_EPI_GLU_BWD: epilogue_tile_act<BLOCK_N, LEANFFN_EPI_GLU_BWD>(LEANFFN_EPI_ARGS); break;
    case LEANFFN_EPI_ACT_BWD: epilogue_tile_act<BLOCK_N, LEANFFN_EPI_ACT_BWD>(LEANFFN_EPI_ARGS); break;
    default: break;
  }
#undef LEANFFN_EPI_ARGS
}

}  // namespace leanffn
