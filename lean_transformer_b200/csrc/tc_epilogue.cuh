// Epilogue of the tcgen05 GEMM kernels.  A warp reads a 32-row x 32-column block of the fp32 accumulator from
// tensor memory (tcgen05.ld gives lane i the 32 columns of row i), transposes it through a private shared-memory
// patch so that four neighbouring lanes own 32 consecutive bytes-or-more of ONE output row, and then applies the
// fused epilogue with fully used 32-byte sectors on every global load and store:
//   lane l, step i (0..3):  row = 8*i + l/4,  columns (l%4)*8 .. +7 of the block.
// Shared by the one-CTA and the CTA-pair kernels; EPI_WARPS warps split the column blocks of a tile.
#pragma once
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace leanffn {

constexpr int EPI_PATCH_FLOATS = 32 * 33;  // per-warp transposition patch (row pitch 33: conflict-free)

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

// One warp's share of a 128-row accumulator tile: TMEM lanes [quarter*32, +32), column blocks
// block_begin, block_begin + block_step, ...  t_acc = TMEM address of (lane quarter*32, first column of the tile);
// row0 = global row of TMEM lane quarter*32; n_blk = tile index along N (gated forward: along the
// intermediate dimension).
template <int BLOCK_N>
__device__ __forceinline__ void epilogue_tile(const EpiParams& ep, int glu_split, uint32_t t_acc, int64_t row0,
                                              int n_blk, bool acc_valid, float* patch, int lane, int block_begin,
                                              int block_step, bool skip_store = false) {
  const int sub_row = lane >> 2;        // + 8*i
  const int sub_col = (lane & 3) * 8;   // within the 32-column block
  if (ep.kind == LEANFFN_EPI_GLU_FWD) {
    if constexpr (BLOCK_N == 256) {
      // tile columns [0,128): gate, [128,256): linear half; output feature j = n_blk*128 + column
      const int inter = glu_split;
#pragma unroll 1
      for (int blk = block_begin; blk < 4; blk += block_step) {
        float g[4][8], l[4][8];
        load_block_transposed(t_acc + blk * 32, patch, lane, acc_valid, g);
        load_block_transposed(t_acc + 128 + blk * 32, patch, lane, acc_valid, l);
        const int64_t j = static_cast<int64_t>(n_blk) * 128 + blk * 32 + sub_col;
        if (j >= inter || skip_store) continue;
        float bg[8] = {0, 0, 0, 0, 0, 0, 0, 0}, bl[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (ep.bias != nullptr) {
          load8(ep.bias, ep.bias_dtype, j, bg);
          load8(ep.bias, ep.bias_dtype, inter + j, bl);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int64_t row = row0 + 8 * i + sub_row;
          if (row >= ep.M) continue;
          float h[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            g[i][q] = bf16_round(g[i][q] + bg[q]);
            l[i][q] = bf16_round(l[i][q] + bl[q]);
            h[q] = bf16_round(act_fwd<true>(ep.act, g[i][q])) * l[i][q];
          }
          store8(ep.D, ep.d_dtype, row * ep.ldd + j, g[i]);
          store8(ep.D, ep.d_dtype, row * ep.ldd + inter + j, l[i]);
          store8(ep.D2, ep.d_dtype, row * ep.ldd2 + j, h);
        }
      }
    }
    return;
  }
#pragma unroll 1
  for (int blk = block_begin; blk < BLOCK_N / 32; blk += block_step) {
    float v[4][8];
    load_block_transposed(t_acc + blk * 32, patch, lane, acc_valid, v);
    const int64_t col = static_cast<int64_t>(n_blk) * BLOCK_N + blk * 32 + sub_col;
    if (col >= ep.N || skip_store) continue;
    float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (ep.bias != nullptr) load8(ep.bias, ep.bias_dtype, col, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t row = row0 + 8 * i + sub_row;
      if (row >= ep.M) continue;
      float(&x)[8] = v[i];
      switch (ep.kind) {
        case LEANFFN_EPI_STORE: {
#pragma unroll
          for (int q = 0; q < 8; ++q) x[q] += b[q];
          store8(ep.D, ep.d_dtype, row * ep.ldd + col, x);
          break;
        }
        case LEANFFN_EPI_ACT_FWD: {
          float h[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            x[q] = bf16_round(x[q] + b[q]);
            h[q] = act_fwd<true>(ep.act, x[q]);
          }
          store8(ep.D, ep.d_dtype, row * ep.ldd + col, x);
          store8(ep.D2, ep.d_dtype, row * ep.ldd2 + col, h);
          break;
        }
        case LEANFFN_EPI_DROPOUT_RESIDUAL: {
#pragma unroll
          for (int q = 0; q < 8; ++q) x[q] += b[q];
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
          if (ep.aux != nullptr) {
            float a[8];
            load8(ep.aux, ep.aux_dtype, row * ep.ldaux + col, a);
#pragma unroll
            for (int q = 0; q < 8; ++q) x[q] += a[q];
          }
          store8(ep.D, ep.d_dtype, row * ep.ldd + col, x);
          break;
        }
        case LEANFFN_EPI_GLU_BWD: {
          // x = dHid[row, col..]; aux = pre [M, 2N]; D = dPre [M, 2N]; D2 = hid [M, N] (optional)
          float g[8], l[8], dl[8];
          load8(ep.aux, ep.aux_dtype, row * ep.ldaux + col, g);
          load8(ep.aux, ep.aux_dtype, row * ep.ldaux + ep.N + col, l);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            float y, d;
            act_fwd_bwd<true>(ep.act, g[q], y, d);
            y = bf16_round(y);
            dl[q] = x[q] * y;        // d/d(linear half)
            g[q] = x[q] * l[q] * d;  // d/d(gate)
            l[q] = y * l[q];         // rematerialised hid
          }
          store8(ep.D, ep.d_dtype, row * ep.ldd + col, g);
          store8(ep.D, ep.d_dtype, row * ep.ldd + ep.N + col, dl);
          if (ep.D2 != nullptr) store8(ep.D2, ep.d_dtype, row * ep.ldd2 + col, l);
          break;
        }
        case LEANFFN_EPI_ACT_BWD: {
          float g[8], h[8];
          load8(ep.aux, ep.aux_dtype, row * ep.ldaux + col, g);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            float y, d;
            act_fwd_bwd<true>(ep.act, g[q], y, d);
            x[q] *= d;
            h[q] = y;
          }
          store8(ep.D, ep.d_dtype, row * ep.ldd + col, x);
          if (ep.D2 != nullptr) store8(ep.D2, ep.d_dtype, row * ep.ldd2 + col, h);
          break;
        }
        default:
          break;
      }
    }
  }
}

}  // namespace leanffn
