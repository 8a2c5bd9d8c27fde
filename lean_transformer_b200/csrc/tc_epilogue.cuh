// Epilogue of the tcgen05 GEMM kernels: reads one 128-row accumulator tile back from tensor memory
// (32 columns per tcgen05.ld) and applies the fused epilogue.  Shared by the one-CTA and the CTA-pair kernels.
#pragma once
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace leanffn {

// ---- epilogue on one 32-column run of one accumulator row --------------------------------------
__device__ __forceinline__ void store_run_bf16(bf16* dst, const float (&v)[32], int ncols_valid) {
  // ncols_valid is a multiple of 8
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    if (q * 8 < ncols_valid) {
      uint4 w;
      w.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
      w.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
      w.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
      w.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
      *reinterpret_cast<uint4*>(dst + q * 8) = w;
    }
  }
}
__device__ __forceinline__ void store_run_f32(float* dst, const float (&v)[32], int ncols_valid) {
#pragma unroll
  for (int q = 0; q < 8; ++q)
    if (q * 4 < ncols_valid)
      *reinterpret_cast<float4*>(dst + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
}
__device__ __forceinline__ void store_run(void* base, int32_t dtype, int64_t elem, const float (&v)[32], int nvalid) {
  if (dtype == LEANFFN_BF16)
    store_run_bf16(static_cast<bf16*>(base) + elem, v, nvalid);
  else
    store_run_f32(static_cast<float*>(base) + elem, v, nvalid);
}
__device__ __forceinline__ void load_run(const void* base, int32_t dtype, int64_t elem, float (&v)[32], int nvalid) {
  if (dtype == LEANFFN_BF16) {
    const bf16* p = static_cast<const bf16*>(base) + elem;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q * 8 < nvalid) {
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(p + q * 8));
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u[h]);
          v[q * 8 + 2 * h] = __low2float(b);
          v[q * 8 + 2 * h + 1] = __high2float(b);
        }
      } else {
#pragma unroll
        for (int h = 0; h < 8; ++h) v[q * 8 + h] = 0.f;
      }
    }
  } else {
    const float* p = static_cast<const float*>(base) + elem;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q * 4 < nvalid) {
        const float4 w = __ldg(reinterpret_cast<const float4*>(p + q * 4));
        v[q * 4] = w.x, v[q * 4 + 1] = w.y, v[q * 4 + 2] = w.z, v[q * 4 + 3] = w.w;
      } else {
        v[q * 4] = v[q * 4 + 1] = v[q * 4 + 2] = v[q * 4 + 3] = 0.f;
      }
    }
  }
}
__device__ __forceinline__ void add_bias(const EpiParams& ep, int64_t col, float (&v)[32], int nvalid) {
  if (ep.bias == nullptr) return;
  float b[32];
  load_run(ep.bias, ep.bias_dtype, col, b, nvalid);
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] += b[j];
}
__device__ __forceinline__ void as_f32(const uint32_t (&r)[32], float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}

// One thread = one accumulator row (TMEM lane).  t_acc: TMEM address of the row's first column;
// n_blk: tile index along N (for the gated forward: along the intermediate dimension).
template <int BLOCK_N>
__device__ __forceinline__ void epilogue_tile(const EpiParams& ep, int glu_split, uint32_t t_acc, int64_t row,
                                              bool row_ok, int n_blk, bool acc_valid) {
  const bool glu_fwd = ep.kind == LEANFFN_EPI_GLU_FWD;
  if (glu_fwd) {
    // columns [0,128): gate, [128,256): linear half; output feature j = n_blk*128 + c
    if constexpr (BLOCK_N == 256) {
      const int inter = glu_split;
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t rg[32], rl[32];
        __syncwarp();
        tmem_ld_32x32(t_acc + c, rg);
        tmem_ld_32x32(t_acc + 128 + c, rl);
        tmem_ld_wait();
        const int64_t j = static_cast<int64_t>(n_blk) * 128 + c;
        const int nvalid = static_cast<int>(inter - j < 32 ? inter - j : 32);
        if (row_ok && nvalid > 0) {
          float g[32], l[32], h[32];
          as_f32(rg, g);
          as_f32(rl, l);
          add_bias(ep, j, g, nvalid);
          add_bias(ep, inter + j, l, nvalid);
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            g[q] = bf16_round(g[q]);
            l[q] = bf16_round(l[q]);
            h[q] = bf16_round(act_fwd<true>(ep.act, g[q])) * l[q];
          }
          store_run(ep.D, ep.d_dtype, row * ep.ldd + j, g, nvalid);
          store_run(ep.D, ep.d_dtype, row * ep.ldd + inter + j, l, nvalid);
          store_run(ep.D2, ep.d_dtype, row * ep.ldd2 + j, h, nvalid);
        }
      }
    }
  } else {
#pragma unroll 1
    for (int c = 0; c < BLOCK_N; c += 32) {
      uint32_t r[32];
      __syncwarp();
      tmem_ld_32x32(t_acc + c, r);
      tmem_ld_wait();
      const int64_t col = static_cast<int64_t>(n_blk) * BLOCK_N + c;
      const int nvalid = static_cast<int>(ep.N - col < 32 ? ep.N - col : 32);
      if (!row_ok || nvalid <= 0) continue;
      float v[32];
      as_f32(r, v);
      if (!acc_valid) {
#pragma unroll
        for (int q = 0; q < 32; ++q) v[q] = 0.f;
      }
      switch (ep.kind) {
        case LEANFFN_EPI_STORE: {
          add_bias(ep, col, v, nvalid);
          store_run(ep.D, ep.d_dtype, row * ep.ldd + col, v, nvalid);
          break;
        }
        case LEANFFN_EPI_ACT_FWD: {
          add_bias(ep, col, v, nvalid);
          float h[32];
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            v[q] = bf16_round(v[q]);
            h[q] = act_fwd<true>(ep.act, v[q]);
          }
          store_run(ep.D, ep.d_dtype, row * ep.ldd + col, v, nvalid);
          store_run(ep.D2, ep.d_dtype, row * ep.ldd2 + col, h, nvalid);
          break;
        }
        case LEANFFN_EPI_DROPOUT_RESIDUAL: {
          add_bias(ep, col, v, nvalid);
          if (ep.threshold != 0u) {
            const uint64_t e0 = ep.elem_offset + static_cast<uint64_t>(row) * ep.N + col;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              bool keep[4];
              dropout_keep4((e0 >> 2) + q, ep.seed, ep.threshold, keep);
#pragma unroll
              for (int h = 0; h < 4; ++h) v[q * 4 + h] = keep[h] ? v[q * 4 + h] * ep.keep_scale : 0.f;
            }
          }
          if (ep.aux != nullptr) {
            float a[32];
            load_run(ep.aux, ep.aux_dtype, row * ep.ldaux + col, a, nvalid);
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] += a[q];
          }
          store_run(ep.D, ep.d_dtype, row * ep.ldd + col, v, nvalid);
          break;
        }
        case LEANFFN_EPI_GLU_BWD: {
          // v = dHid[row, col..]; aux = pre [M, 2N]; D = dPre [M, 2N]; D2 = hid [M, N] (optional)
          float g[32], l[32], dl[32];
          load_run(ep.aux, ep.aux_dtype, row * ep.ldaux + col, g, nvalid);
          load_run(ep.aux, ep.aux_dtype, row * ep.ldaux + ep.N + col, l, nvalid);
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            float y, d;
            act_fwd_bwd<true>(ep.act, g[q], y, d);
            y = bf16_round(y);
            dl[q] = v[q] * y;        // d/d(linear half)
            g[q] = v[q] * l[q] * d;  // d/d(gate)
            l[q] = y * l[q];         // rematerialised hid
          }
          store_run(ep.D, ep.d_dtype, row * ep.ldd + col, g, nvalid);
          store_run(ep.D, ep.d_dtype, row * ep.ldd + ep.N + col, dl, nvalid);
          if (ep.D2 != nullptr) store_run(ep.D2, ep.d_dtype, row * ep.ldd2 + col, l, nvalid);
          break;
        }
        case LEANFFN_EPI_ACT_BWD: {
          float g[32], h[32];
          load_run(ep.aux, ep.aux_dtype, row * ep.ldaux + col, g, nvalid);
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            float y, d;
            act_fwd_bwd<true>(ep.act, g[q], y, d);
            v[q] *= d;
            h[q] = y;
          }
          store_run(ep.D, ep.d_dtype, row * ep.ldd + col, v, nvalid);
          if (ep.D2 != nullptr) store_run(ep.D2, ep.d_dtype, row * ep.ldd2 + col, h, nvalid);
          break;
        }
        default:
          break;
      }
    }
  }
}

}  // namespace leanffn
