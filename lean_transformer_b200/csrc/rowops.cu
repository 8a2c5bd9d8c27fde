// HBM-bound row / elementwise kernels of the LeanFFN path: LayerNorm forward and backward,
// (gated) activation forward / backward, dropout, column sums (bias gradients), casts, transposes.
// All of them move each element across HBM once per pass with 8- or 16-byte accesses and reduce
// within rows by warp shuffles; grids are sized in multiples of the SM count.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gemm_common.cuh"

namespace leanffn {

static int g_sm_count_cache[64] = {0};
int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (g_sm_count_cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count_cache[dev] = n;
  }
  return g_sm_count_cache[dev];
}

static inline int32_t launch_status() {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LEANFFN_OK : 1000 + static_cast<int32_t>(e);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the WPR warps that share one row. WPR == 1: warp shuffle only.
template <int WPR>
__device__ __forceinline__ float row_sum(float v, float* smem, int row_in_block, int warp_in_row, int lane) {
  v = warp_sum(v);
  if constexpr (WPR > 1) {
    __syncthreads();  // protect smem reuse between consecutive reductions
    if (lane == 0) smem[row_in_block * WPR + warp_in_row] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) t += smem[row_in_block * WPR + w];
    v = t;
  }
  return v;
}

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Pair of sums over the WPR warps of one row with ONE block barrier: callers alternate between two shared buffers
// (`parity`), so a buffer is rewritten only after a later barrier has seen every reader leave it.
template <int WPR>
__device__ __forceinline__ float2 row_sum_pair(float a, float b, float2* buffers, int buffer_len, int& parity,
                                               int row_in_block, int warp_in_row, int lane) {
  a = warp_sum(a);
  b = warp_sum(b);
  if constexpr (WPR > 1) {
    float2* buf = buffers + parity * buffer_len + row_in_block * WPR;
    parity ^= 1;
    if (lane == 0) buf[warp_in_row] = make_float2(a, b);
    __syncthreads();
    const float2 t = lane < WPR ? buf[lane] : make_float2(0.f, 0.f);
    a = warp_sum(t.x);
    b = warp_sum(t.y);
  }
  return make_float2(a, b);
}

constexpr int LN_THREADS = 256;

// ---- LayerNorm forward ---------------------------------------------------------------------
// A row is held in registers by WPR warps (VPT 4-element vectors per thread); mean and the
// variance about that mean are two separate reductions, so constant rows give var == 0 exactly.
template <typename TX, typename TP, typename TY, typename TR, int VPT, int WPR>
__global__ void __launch_bounds__(LN_THREADS)
ln_fwd_kernel(const TX* __restrict__ x, const TP* __restrict__ gamma, const TP* __restrict__ beta, TY* __restrict__ y,
              const TR* __restrict__ residual, int64_t rows, int cols, float eps, uint32_t threshold, float keep_scale,
              uint64_t seed, uint64_t elem_offset) {
  constexpr int ROWS_PER_BLOCK = (LN_THREADS / 32) / WPR;
  __shared__ float red[LN_THREADS / 32];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row_in_block = warp / WPR;
  const int warp_in_row = warp % WPR;
  const int t_in_row = warp_in_row * 32 + lane;
  const float inv_cols = 1.0f / static_cast<float>(cols);

  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * ROWS_PER_BLOCK; row0 < rows;
       row0 += static_cast<int64_t>(gridDim.x) * ROWS_PER_BLOCK) {
    const int64_t row = row0 + row_in_block;
    const bool row_ok = row < rows;
    float v[VPT][4];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = (t_in_row + i * 32 * WPR) * 4;
      if (row_ok && c < cols) {
        Vec4<TX> q;
        q.load(x + row * cols + c);
        q.get(v[i]);
      } else {
        v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
      }
      s += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
    }
    const float mean = row_sum<WPR>(s, red, row_in_block, warp_in_row, lane) * inv_cols;
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = (t_in_row + i * 32 * WPR) * 4;
      if (c < cols) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float d = v[i][j] - mean;
          s2 += d * d;
        }
      }
    }
    const float var = row_sum<WPR>(s2, red, row_in_block, warp_in_row, lane) * inv_cols;
    const float rstd = rsqrtf(var + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = (t_in_row + i * 32 * WPR) * 4;
      if (row_ok && c < cols) {
        float g[4] = {1.f, 1.f, 1.f, 1.f}, b[4] = {0.f, 0.f, 0.f, 0.f}, o[4];
        if (gamma != nullptr) {
          Vec4<TP> q;
          q.load(gamma + c);
          q.get(g);
        }
        if (beta != nullptr) {
          Vec4<TP> q;
          q.load(beta + c);
          q.get(b);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = (v[i][j] - mean) * rstd * g[j] + b[j];
        if (threshold != 0u) {
          bool keep[4];
          dropout_keep4((elem_offset + static_cast<uint64_t>(row) * cols + c) >> 2, seed, threshold, keep);
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = keep[j] ? o[j] * keep_scale : 0.f;
        }
        if (residual != nullptr) {
          Vec4<TR> q;
          float r[4];
          q.load(residual + row * cols + c);
          q.get(r);
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] += r[j];
        }
        Vec4<TY> out;
        out.set(o);
        out.store(y + row * cols + c);
      }
    }
  }
}

// Any column count (not a multiple of 4, or wider than the register path): one block per row,
// three passes over the row (L1/L2 resident after the first).
template <typename TX, typename TP, typename TY, typename TR>
__global__ void __launch_bounds__(LN_THREADS)
ln_fwd_generic_kernel(const TX* __restrict__ x, const TP* __restrict__ gamma, const TP* __restrict__ beta,
                      TY* __restrict__ y, const TR* __restrict__ residual, int64_t rows, int cols, float eps,
                      uint32_t threshold, float keep_scale, uint64_t seed, uint64_t elem_offset) {
  __shared__ float red[LN_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_cols = 1.0f / static_cast<float>(cols);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const TX* xr = x + row * cols;
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += LN_THREADS) s += to_f32(xr[c]);
    const float mean = row_sum<LN_THREADS / 32>(s, red, 0, warp, lane) * inv_cols;
    float s2 = 0.f;
    for (int c = threadIdx.x; c < cols; c += LN_THREADS) {
      const float d = to_f32(xr[c]) - mean;
      s2 += d * d;
    }
    const float rstd = rsqrtf(row_sum<LN_THREADS / 32>(s2, red, 0, warp, lane) * inv_cols + eps);
    for (int c = threadIdx.x; c < cols; c += LN_THREADS) {
      float o = (to_f32(xr[c]) - mean) * rstd * (gamma ? to_f32(gamma[c]) : 1.f) + (beta ? to_f32(beta[c]) : 0.f);
      if (threshold != 0u)
        o = dropout_keep1(elem_offset + static_cast<uint64_t>(row) * cols + c, seed, threshold) ? o * keep_scale : 0.f;
      if (residual != nullptr) o += to_f32(residual[row * cols + c]);
      y[row * cols + c] = from_f32<TY>(o);
    }
  }
}

// ---- LayerNorm backward --------------------------------------------------------------------
// Partial dgamma / dbeta of the rows a (block, row-slot) pair visits go to
// part[(blockIdx.x * ROWS_PER_BLOCK + row_in_block) * 2 * cols + {0, cols} + c]; a column-sum pass
// finishes them.
// Wide rows are spread over up to 32 warps (1024 threads) so that a thread keeps few values and the SM many warps:
// the kernel is a chain of load -> four row reductions -> store per row, and only other warps hide that latency.
__host__ __device__ constexpr int ln_bwd_threads(int wpr) { return wpr > LN_THREADS / 32 ? wpr * 32 : LN_THREADS; }

template <typename TD, typename TX, typename TP, typename TR, typename TO, int VPT, int WPR>
__global__ void __launch_bounds__(ln_bwd_threads(WPR))
ln_bwd_kernel(const TD* __restrict__ dy, const TX* __restrict__ x, const TP* __restrict__ gamma,
              const TR* __restrict__ dres, TO* __restrict__ dx, float* __restrict__ part, int64_t rows, int cols,
              float eps) {
  constexpr int THREADS = ln_bwd_threads(WPR);
  constexpr int ROWS_PER_BLOCK = (THREADS / 32) / WPR;
  __shared__ float2 red[2 * (THREADS / 32)];
  int parity = 0;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row_in_block = warp / WPR;
  const int warp_in_row = warp % WPR;
  const int t_in_row = warp_in_row * 32 + lane;
  const float inv_cols = 1.0f / static_cast<float>(cols);

  float acc_g[VPT][4], acc_b[VPT][4];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_g[i][j] = acc_b[i][j] = 0.f;

  // One row's operands in registers.  Variants with few values per thread keep TWO rows: the loads of the next row are issued
  // before the reductions of the current one, which doubles the bytes each thread has in flight (the kernel is a
  // chain of dependent block reductions per row, so nothing else hides the memory latency).
  struct RowData {
    float v[VPT][4], d[VPT][4];
    Vec4<TR> res[VPT];  // residual gradient, requested together with x and dy (one memory round trip per row)
  };
  const int64_t stride = static_cast<int64_t>(gridDim.x) * ROWS_PER_BLOCK;
  const bool use_res = dres != nullptr && dx != nullptr;
  auto load_row = [&](RowData& r, int64_t row0) {
    const int64_t row = row0 + row_in_block;
    const bool row_ok = row < rows;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = (t_in_row + i * 32 * WPR) * 4;
      if (row_ok && c < cols) {
        Vec4<TX> q;
        q.load(x + row * cols + c);
        q.get(r.v[i]);
        Vec4<TD> qd;
        qd.load(dy + row * cols + c);
        qd.get(r.d[i]);
        if (use_res) r.res[i].load(dres + row * cols + c);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) r.v[i][j] = r.d[i][j] = 0.f;
      }
    }
  };
  auto prefetch_row = [&](int64_t row0) {
    // the row this thread visits after the ones held in registers goes to L2 now
    const int64_t next = row0 + row_in_block;
    if (next < rows) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = (t_in_row + i * 32 * WPR) * 4;
        if (c < cols) {
          prefetch_l2(x + next * cols + c);
          prefetch_l2(dy + next * cols + c);
          if (use_res) prefetch_l2(dres + next * cols + c);
        }
      }
    }
  };
  auto process_row = [&](RowData& r, int64_t row0) {
    const int64_t row = row0 + row_in_block;
    const bool row_ok = row < rows;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) s += (r.v[i][0] + r.v[i][1]) + (r.v[i][2] + r.v[i][3]);
    const float mean = row_sum_pair<WPR>(s, 0.f, red, THREADS / 32, parity, row_in_block, warp_in_row, lane).x * inv_cols;
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = (t_in_row + i * 32 * WPR) * 4;
      if (c < cols) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float t = r.v[i][j] - mean;
          s2 += t * t;
        }
      }
    }
    const float rstd =
        rsqrtf(row_sum_pair<WPR>(s2, 0.f, red, THREADS / 32, parity, row_in_block, warp_in_row, lane).x * inv_cols + eps);
    // v <- normalised x, d stays dy; g = dy * gamma
    float sg = 0.f, sgx = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = (t_in_row + i * 32 * WPR) * 4;
      float g[4] = {1.f, 1.f, 1.f, 1.f};
      if (gamma != nullptr && c < cols) {
        Vec4<TP> q;
        q.load(gamma + c);
        q.get(g);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float xn = (c < cols && row_ok) ? (r.v[i][j] - mean) * rstd : 0.f;
        r.v[i][j] = xn;
        acc_g[i][j] += r.d[i][j] * xn;
        acc_b[i][j] += r.d[i][j];
        r.d[i][j] *= g[j];
        sg += r.d[i][j];
        sgx += r.d[i][j] * xn;
      }
    }
    const float2 sums = row_sum_pair<WPR>(sg, sgx, red, THREADS / 32, parity, row_in_block, warp_in_row, lane);
    const float mg = sums.x * inv_cols, mgx = sums.y * inv_cols;
    if (dx != nullptr) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = (t_in_row + i * 32 * WPR) * 4;
        if (row_ok && c < cols) {
          float o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = rstd * (r.d[i][j] - mg - r.v[i][j] * mgx);
          if (dres != nullptr) {
            float rr[4];
            r.res[i].get(rr);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] += rr[j];
          }
          Vec4<TO> out;
          out.set(o);
          out.store(dx + row * cols + c);
        }
      }
    }
  };

  int64_t row0 = static_cast<int64_t>(blockIdx.x) * ROWS_PER_BLOCK;
  if constexpr (VPT <= 2 && WPR <= 16) {  // 1024-thread blocks have 64 registers per thread: no room for two rows
    RowData a, b;
    if (row0 < rows) load_row(a, row0);
    while (row0 < rows) {
      if (row0 + stride < rows) load_row(b, row0 + stride);
      prefetch_row(row0 + 2 * stride);
      process_row(a, row0);
      row0 += stride;
      if (row0 >= rows) break;
      if (row0 + stride < rows) load_row(a, row0 + stride);
      prefetch_row(row0 + 2 * stride);
      process_row(b, row0);
      row0 += stride;
    }
  } else {
    RowData a;
    for (; row0 < rows; row0 += stride) {
      prefetch_row(row0 + stride);
      load_row(a, row0);
      process_row(a, row0);
    }
  }
  if (part != nullptr) {
    float* p = part + (static_cast<int64_t>(blockIdx.x) * ROWS_PER_BLOCK + row_in_block) * 2 * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = (t_in_row + i * 32 * WPR) * 4;
      if (c < cols) {
        *reinterpret_cast<float4*>(p + c) = make_float4(acc_g[i][0], acc_g[i][1], acc_g[i][2], acc_g[i][3]);
        *reinterpret_cast<float4*>(p + cols + c) = make_float4(acc_b[i][0], acc_b[i][1], acc_b[i][2], acc_b[i][3]);
      }
    }
  }
}

// Generic-width backward: one block per row slot, partials accumulated in global scratch rows.
template <typename TD, typename TX, typename TP, typename TR, typename TO>
__global__ void __launch_bounds__(LN_THREADS)
ln_bwd_generic_kernel(const TD* __restrict__ dy, const TX* __restrict__ x, const TP* __restrict__ gamma,
                      const TR* __restrict__ dres, TO* __restrict__ dx, float* __restrict__ part, int64_t rows,
                      int cols, float eps) {
  __shared__ float red[LN_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_cols = 1.0f / static_cast<float>(cols);
  float* p = part ? part + static_cast<int64_t>(blockIdx.x) * 2 * cols : nullptr;
  if (p != nullptr)
    for (int c = threadIdx.x; c < 2 * cols; c += LN_THREADS) p[c] = 0.f;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const TX* xr = x + row * cols;
    const TD* dr = dy + row * cols;
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += LN_THREADS) s += to_f32(xr[c]);
    const float mean = row_sum<LN_THREADS / 32>(s, red, 0, warp, lane) * inv_cols;
    float s2 = 0.f;
    for (int c = threadIdx.x; c < cols; c += LN_THREADS) {
      const float t = to_f32(xr[c]) - mean;
      s2 += t * t;
    }
    const float rstd = rsqrtf(row_sum<LN_THREADS / 32>(s2, red, 0, warp, lane) * inv_cols + eps);
    float sg = 0.f, sgx = 0.f;
    for (int c = threadIdx.x; c < cols; c += LN_THREADS) {
      const float xn = (to_f32(xr[c]) - mean) * rstd;
      const float g = to_f32(dr[c]) * (gamma ? to_f32(gamma[c]) : 1.f);
      sg += g;
      sgx += g * xn;
    }
    const float mg = row_sum<LN_THREADS / 32>(sg, red, 0, warp, lane) * inv_cols;
    const float mgx = row_sum<LN_THREADS / 32>(sgx, red, 0, warp, lane) * inv_cols;
    for (int c = threadIdx.x; c < cols; c += LN_THREADS) {
      const float xn = (to_f32(xr[c]) - mean) * rstd;
      const float dyv = to_f32(dr[c]);
      if (p != nullptr) {
        p[c] += dyv * xn;  // column c is owned by this thread for the whole kernel
        p[cols + c] += dyv;
      }
      if (dx != nullptr) {
        float o = rstd * (dyv * (gamma ? to_f32(gamma[c]) : 1.f) - mg - xn * mgx);
        if (dres != nullptr) o += to_f32(dres[row * cols + c]);
        dx[row * cols + c] = from_f32<TO>(o);
      }
    }
  }
}

// ---- column sums ------------------------------------------------------------------------------
// Block = 32 column lanes (4 columns each) x 8 row lanes; grid = (ceil(cols/128), chunks).
// out[chunk * out_stride + c] = sum over the chunk's rows.  vec_ok (decided on the host from the base address
// and the leading dimension) allows 4-element vector loads; otherwise every element is loaded on its own.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_kernel(const T* __restrict__ x, int64_t ld, float* __restrict__ out, int64_t out_stride, int64_t rows,
              int64_t cols, int64_t rows_per_chunk, int vec_ok) {
  __shared__ float sm[8][132];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int64_t c = (static_cast<int64_t>(blockIdx.x) * 32 + cx) * 4;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_chunk;
  const int64_t r1 = min(rows, r0 + rows_per_chunk);
  float a[4] = {0.f, 0.f, 0.f, 0.f};
  if (c + 3 < cols && vec_ok) {
    for (int64_t r = r0 + ry; r < r1; r += 8) {
      Vec4<T> q;
      float f[4];
      q.load(x + r * ld + c);
      q.get(f);
#pragma unroll
      for (int j = 0; j < 4; ++j) a[j] += f[j];
    }
  } else {
    for (int64_t r = r0 + ry; r < r1; r += 8)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j < cols) a[j] += to_f32(x[r * ld + c + j]);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) sm[ry][cx * 4 + j] = a[j];
  __syncthreads();
  if (threadIdx.x < 128) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sm[k][threadIdx.x];
    const int64_t cc = static_cast<int64_t>(blockIdx.x) * 128 + threadIdx.x;
    if (cc < cols) out[static_cast<int64_t>(blockIdx.y) * out_stride + cc] = t;
  }
}

static int64_t colsum_chunks(int64_t rows, int64_t cols) {
  const int64_t col_blocks = (cols + 127) / 128;
  int64_t chunks = (static_cast<int64_t>(sm_count()) * 8 + col_blocks - 1) / col_blocks;
  const int64_t max_chunks = (rows + 63) / 64;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  return chunks;
}

template <typename T>
static int32_t colsum_launch(const T* x, int64_t ld, float* out, float* scratch, int64_t rows, int64_t cols,
                             cudaStream_t st) {
  const int64_t chunks = colsum_chunks(rows, cols);
  const dim3 grid1(static_cast<unsigned>((cols + 127) / 128), static_cast<unsigned>(chunks));
  // a row of 4 elements is loaded as one vector only if every such vector is naturally aligned
  const int vec1 = (ld % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % (4 * sizeof(T)) == 0);
  if (chunks == 1) {
    colsum_kernel<T><<<grid1, 256, 0, st>>>(x, ld, out, cols, rows, cols, rows, vec1);
    return launch_status();
  }
  const int64_t rpc = (rows + chunks - 1) / chunks;
  colsum_kernel<T><<<grid1, 256, 0, st>>>(x, ld, scratch, cols, rows, cols, rpc, vec1);
  const dim3 grid2(static_cast<unsigned>((cols + 127) / 128), 1);
  const int vec2 = (cols % 4 == 0) && (reinterpret_cast<uintptr_t>(scratch) % 16 == 0);
  colsum_kernel<float><<<grid2, 256, 0, st>>>(scratch, cols, out, cols, chunks, cols, chunks, vec2);
  return launch_status();
}

int32_t launch_colsum_into_partials(const void* x, int32_t dtype, int64_t ld, float* partial, int64_t ld_partial,
                                    int64_t rows, int64_t cols, cudaStream_t st) {
  const int64_t groups = (rows + 31) / 32;
  if (groups > 1) {
    const cudaError_t e = cudaMemset2DAsync(partial + ld_partial, sizeof(float) * ld_partial, 0, sizeof(float) * cols,
                                            static_cast<size_t>(groups - 1), st);
    if (e != cudaSuccess) return 1000 + static_cast<int32_t>(e);
  }
  const dim3 grid(static_cast<unsigned>((cols + 127) / 128), 1);
  if (dtype == LEANFFN_BF16) {
    const int vec = (ld % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 8 == 0);
    colsum_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ld, partial, ld_partial, rows, cols, rows, vec);
  } else {
    const int vec = (ld % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
    colsum_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), ld, partial, ld_partial, rows, cols, rows, vec);
  }
  return launch_status();
}

// ---- activation forward / backward -------------------------------------------------------------
template <typename T, bool FAST>
__global__ void __launch_bounds__(256)
act_fwd_kernel(const T* __restrict__ pre, T* __restrict__ hid, int64_t rows, int64_t inter, int gated, int act) {
  const int64_t vec_per_row = inter / 4;
  const int64_t total = rows * vec_per_row;
  const int64_t ldp = gated ? 2 * inter : inter;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * 4;
    Vec4<T> q;
    float g[4], o[4];
    q.load(pre + r * ldp + c);
    q.get(g);
    if (gated) {
      float l[4];
      q.load(pre + r * ldp + inter + c);
      q.get(l);
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = to_f32(from_f32<T>(act_fwd<FAST>(act, g[j]))) * l[j];
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = act_fwd<FAST>(act, g[j]);
    }
    q.set(o);
    q.store(hid + r * inter + c);
  }
}

template <typename T, bool FAST>
__global__ void __launch_bounds__(256)
act_bwd_kernel(const T* dhid, int64_t ld_dhid, const T* __restrict__ pre, T* dpre, T* __restrict__ hid_out,
               int64_t rows, int64_t inter, int gated, int act) {
  const int64_t vec_per_row = inter / 4;
  const int64_t total = rows * vec_per_row;
  const int64_t ldp = gated ? 2 * inter : inter;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * 4;
    Vec4<T> q;
    float g[4], dh[4], dg[4], h[4];
    q.load(pre + r * ldp + c);
    q.get(g);
    q.load(dhid + r * ld_dhid + c);
    q.get(dh);
    if (gated) {
      float l[4], dl[4];
      q.load(pre + r * ldp + inter + c);
      q.get(l);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float y, d;
        act_fwd_bwd<FAST>(act, g[j], y, d);
        // every product of two stored tensors is rounded to the tensors' type (bf16: as the GEMM epilogue's packed
        // products do), so the fused and the stand-alone formulations agree bit for bit
        y = to_f32(from_f32<T>(y));
        dl[j] = dh[j] * y;
        dg[j] = to_f32(from_f32<T>(dh[j] * l[j])) * to_f32(from_f32<T>(d));
        h[j] = y * l[j];
      }
      q.set(dl);
      q.store(dpre + r * ldp + inter + c);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float y, d;
        act_fwd_bwd<FAST>(act, g[j], y, d);
        dg[j] = dh[j] * to_f32(from_f32<T>(d));
        h[j] = y;
      }
    }
    q.set(dg);
    q.store(dpre + r * ldp + c);
    if (hid_out != nullptr) {
      q.set(h);
      q.store(hid_out + r * inter + c);
    }
  }
}

// ---- dropout, mask, cast ------------------------------------------------------------------------
template <typename TX, typename TY, typename TR>
__global__ void __launch_bounds__(256)
dropout_kernel(const TX* __restrict__ x, TY* __restrict__ y, const TR* __restrict__ residual, int64_t n,
               uint32_t threshold, float keep_scale, uint64_t seed, uint64_t elem_offset, int vec_ok) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nvec = vec_ok ? n / 4 : 0;
  for (int64_t i = tid; i < nvec; i += stride) {
    Vec4<TX> q;
    float f[4];
    q.load(x + i * 4);
    q.get(f);
    if (threshold != 0u) {
      bool keep[4];
      dropout_keep4((elem_offset >> 2) + static_cast<uint64_t>(i), seed, threshold, keep);
#pragma unroll
      for (int j = 0; j < 4; ++j) f[j] = keep[j] ? f[j] * keep_scale : 0.f;
    }
    if (residual != nullptr) {
      Vec4<TR> qr;
      float r[4];
      qr.load(residual + i * 4);
      qr.get(r);
#pragma unroll
      for (int j = 0; j < 4; ++j) f[j] += r[j];
    }
    Vec4<TY> o;
    o.set(f);
    o.store(y + i * 4);
  }
  for (int64_t i = nvec * 4 + tid; i < n; i += stride) {
    float f = to_f32(x[i]);
    if (threshold != 0u) f = dropout_keep1(elem_offset + i, seed, threshold) ? f * keep_scale : 0.f;
    if (residual != nullptr) f += to_f32(residual[i]);
    y[i] = from_f32<TY>(f);
  }
}

// y = dropout(x) cast to TY, and partial[chunk, c] = sum over the chunk's rows of the ROUNDED y[r, c]: the incoming
// gradient of the block is masked, cast and column-summed (bias gradient of the output projection) in one pass.
// Block = 8 warps; a lane owns 8 consecutive columns (16-byte accesses for bf16), the warps stride over the rows of
// the chunk; grid = (cols / 256 rounded up, chunks).  Needs cols % 8 == 0, 16-byte aligned x / y, elem_offset % 4 == 0.
template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
dropout_colsum_kernel(const TX* __restrict__ x, TY* __restrict__ y, float* __restrict__ partial, int64_t rows,
                      int64_t cols, int64_t rows_per_chunk, uint32_t threshold, float keep_scale, uint64_t seed,
                      uint64_t elem_offset) {
  __shared__ float sm[8][264];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c = (static_cast<int64_t>(blockIdx.x) * 32 + lane) * 8;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_chunk;
  const int64_t r1 = min(rows, r0 + rows_per_chunk);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c < cols) {
    for (int64_t r = r0 + warp; r < r1; r += 8) {
      float f[8];
      Vec4<TX> q0, q1;
      q0.load(x + r * cols + c);
      q1.load(x + r * cols + c + 4);
      float a[4], b[4];
      q0.get(a);
      q1.get(b);
#pragma unroll
      for (int j = 0; j < 4; ++j) f[j] = a[j], f[4 + j] = b[j];
      if (threshold != 0u) {
        const uint64_t e0 = elem_offset + static_cast<uint64_t>(r) * cols + c;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          bool keep[4];
          dropout_keep4((e0 >> 2) + h, seed, threshold, keep);
#pragma unroll
          for (int j = 0; j < 4; ++j) f[4 * h + j] = keep[j] ? f[4 * h + j] * keep_scale : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = to_f32(from_f32<TY>(f[j]));
        acc[j] += f[j];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) a[j] = f[j], b[j] = f[4 + j];
      Vec4<TY> o0, o1;
      o0.set(a);
      o1.set(b);
      o0.store(y + r * cols + c);
      o1.store(y + r * cols + c + 4);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sm[k][threadIdx.x];
    const int64_t cc = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (cc < cols) partial[static_cast<int64_t>(blockIdx.y) * cols + cc] = t;
  }
}

static int64_t dropout_colsum_chunks(int64_t rows, int64_t cols) {
  const int64_t col_blocks = (cols + 255) / 256;
  int64_t chunks = (static_cast<int64_t>(sm_count()) * 4 + col_blocks - 1) / col_blocks;
  const int64_t max_chunks = (rows + 15) / 16;
  if (chunks > max_chunks) chunks = max_chunks;
  return chunks < 1 ? 1 : chunks;
}

__global__ void __launch_bounds__(256)
dropout_mask_kernel(uint8_t* __restrict__ mask, int64_t n, uint32_t threshold, uint64_t seed, uint64_t elem_offset) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    mask[i] = dropout_keep1(elem_offset + i, seed, threshold) ? 1 : 0;
}

// ---- transpose ----------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
transpose_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y, int64_t rows, int64_t cols) {
  __shared__ T tile[64][65];
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 64, r0 = static_cast<int64_t>(blockIdx.y) * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int i = ty; i < 64; i += 4) {
    const int64_t r = r0 + i, c = c0 + tx;
    if (r < rows && c < cols) tile[i][tx] = x[r * ldx + c];
  }
  __syncthreads();
  for (int i = ty; i < 64; i += 4) {
    const int64_t c = c0 + i, r = r0 + tx;
    if (r < rows && c < cols) y[c * rows + r] = tile[tx][i];
  }
}

static int grid_for(int64_t work_items, int threads) {
  const int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// ---- dispatch helpers ---------------------------------------------------------------------------
template <typename TX, typename TP, typename TY, typename TR>
static int32_t ln_fwd_dispatch(const void* x, const void* gamma, const void* beta, void* y, const void* residual,
                               int64_t rows, int64_t cols, float eps, uint32_t thr, float ks, uint64_t seed,
                               uint64_t off, cudaStream_t st) {
  const TX* xp = static_cast<const TX*>(x);
  const TP* gp = static_cast<const TP*>(gamma);
  const TP* bp = static_cast<const TP*>(beta);
  TY* yp = static_cast<TY*>(y);
  const TR* rp = static_cast<const TR*>(residual);
  const int c = static_cast<int>(cols);
  const int sms = sm_count();
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  // the register path moves 4-element vectors: every pointer 16-byte aligned, else the scalar kernel below
  const bool vec = (cols % 4 == 0) && (thr == 0u || off % 4 == 0) && al16(x) && al16(y) && al16(gamma) && al16(beta) &&
                   al16(residual);
#define LN_FWD_CASE(VPT, WPR)                                                                                       \
  {                                                                                                                 \
    constexpr int RPB = (LN_THREADS / 32) / WPR;                                                                    \
    int64_t blocks = (rows + RPB - 1) / RPB;                                                                        \
    if (blocks > static_cast<int64_t>(sms) * 8) blocks = static_cast<int64_t>(sms) * 8;                             \
    ln_fwd_kernel<TX, TP, TY, TR, VPT, WPR><<<static_cast<unsigned>(blocks), LN_THREADS, 0, st>>>(                  \
        xp, gp, bp, yp, rp, rows, c, eps, thr, ks, seed, off);                                                      \
    return launch_status();                                                                                         \
  }
  if (vec && cols <= 128) LN_FWD_CASE(1, 1)
  if (vec && cols <= 256) LN_FWD_CASE(2, 1)
  if (vec && cols <= 512) LN_FWD_CASE(4, 1)
  if (vec && cols <= 1024) LN_FWD_CASE(8, 1)
  if (vec && cols <= 2048) LN_FWD_CASE(2, 8)
  if (vec && cols <= 4096) LN_FWD_CASE(4, 8)
  if (vec && cols <= 8192) LN_FWD_CASE(8, 8)
  if (vec && cols <= 16384) LN_FWD_CASE(16, 8)
#undef LN_FWD_CASE
  int64_t blocks = rows < static_cast<int64_t>(sms) * 8 ? rows : static_cast<int64_t>(sms) * 8;
  if (blocks < 1) blocks = 1;
  ln_fwd_generic_kernel<TX, TP, TY, TR><<<static_cast<unsigned>(blocks), LN_THREADS, 0, st>>>(
      xp, gp, bp, yp, rp, rows, c, eps, thr, ks, seed, off);
  return launch_status();
}

struct LnBwdPlan {
  int vpt, wpr;       // 0,0 => generic kernel
  int64_t blocks;     // grid size
  int64_t part_rows;  // rows of the [part_rows, 2*cols] partial buffer
};
static LnBwdPlan ln_bwd_plan(int64_t rows, int64_t cols) {
  LnBwdPlan p{0, 0, 0, 0};
  const int sms = sm_count();
  if (cols % 4 == 0 && cols <= 16384) {
    if (cols <= 128) p.vpt = 1, p.wpr = 1;
    else if (cols <= 256) p.vpt = 2, p.wpr = 1;
    else if (cols <= 512) p.vpt = 4, p.wpr = 1;
    else if (cols <= 1024) p.vpt = 2, p.wpr = 4;  // (one warp per row, 8 vectors per thread: measured 8 % slower)
    else if (cols <= 2048) p.vpt = 2, p.wpr = 8;
    else if (cols <= 4096) p.vpt = 2, p.wpr = 16;
    else if (cols <= 8192) p.vpt = 2, p.wpr = 32;
    else p.vpt = 16, p.wpr = 8;
    const int threads = ln_bwd_threads(p.wpr);
    const int rpb = (threads / 32) / p.wpr;
    int64_t blocks = (rows + rpb - 1) / rpb;
    // co-resident blocks per SM: the 2-vector variants use 64 registers per thread
    const int per_sm = p.vpt <= 2 ? 1024 / threads : 2;
    const int64_t cap = static_cast<int64_t>(sms) * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    p.blocks = blocks;
    p.part_rows = blocks * rpb;
  } else {
    int64_t blocks = rows < static_cast<int64_t>(sms) * 2 ? rows : static_cast<int64_t>(sms) * 2;
    if (blocks < 1) blocks = 1;
    p.blocks = blocks;
    p.part_rows = blocks;
  }
  return p;
}

template <typename TD, typename TX, typename TP, typename TR, typename TO>
static int32_t ln_bwd_dispatch(const void* dy, const void* x, const void* gamma, const void* dres, void* dx,
                               float* dgamma, float* dbeta, void* scratch, int64_t rows, int64_t cols, float eps,
                               cudaStream_t st) {
  const LnBwdPlan plan = ln_bwd_plan(rows, cols);
  const TD* dyp = static_cast<const TD*>(dy);
  const TX* xp = static_cast<const TX*>(x);
  const TP* gp = static_cast<const TP*>(gamma);
  const TR* rp = static_cast<const TR*>(dres);
  TO* dxp = static_cast<TO*>(dx);
  float* part = (dgamma != nullptr) ? static_cast<float*>(scratch) : nullptr;
  const int c = static_cast<int>(cols);
  const unsigned grid = static_cast<unsigned>(plan.blocks);
#define LN_BWD_CASE(VPT, WPR)                                                                                  \
  if (plan.vpt == VPT && plan.wpr == WPR)                                                                      \
    ln_bwd_kernel<TD, TX, TP, TR, TO, VPT, WPR><<<grid, ln_bwd_threads(WPR), 0, st>>>(dyp, xp, gp, rp, dxp, part, \
                                                                                     rows, c, eps);
  LN_BWD_CASE(1, 1)
  else LN_BWD_CASE(2, 1)
  else LN_BWD_CASE(4, 1)
  else LN_BWD_CASE(2, 4)
  else LN_BWD_CASE(2, 8)
  else LN_BWD_CASE(2, 16)
  else LN_BWD_CASE(2, 32)
  else LN_BWD_CASE(16, 8)
  else ln_bwd_generic_kernel<TD, TX, TP, TR, TO><<<grid, LN_THREADS, 0, st>>>(dyp, xp, gp, rp, dxp, part, rows, c, eps);
#undef LN_BWD_CASE
  int32_t s = launch_status();
  if (s != LEANFFN_OK || part == nullptr) return s;
  // finish: [part_rows, 2*cols] -> dgamma | dbeta (written as one [2*cols] vector when contiguous)
  float* tail = part + plan.part_rows * 2 * cols;  // second-stage scratch
  s = colsum_launch<float>(part, 2 * cols, tail + 0, tail + 2 * cols, plan.part_rows, 2 * cols, st);
  if (s != LEANFFN_OK) return s;
  cudaMemcpyAsync(dgamma, tail, sizeof(float) * cols, cudaMemcpyDeviceToDevice, st);
  cudaMemcpyAsync(dbeta, tail + cols, sizeof(float) * cols, cudaMemcpyDeviceToDevice, st);
  return launch_status();
}

// ---- barrier between ranks over peer-mapped flag words ---------------------------------------------------------
struct PeerBarrierArgs {
  uint32_t* flags[8];
  int32_t rank, world, channel;
  uint32_t epoch;
  long long limit;
  int32_t* status;
};

__global__ void __launch_bounds__(32)
peer_barrier_kernel(const PeerBarrierArgs a) {
  const int t = threadIdx.x;
  if (t < a.world && t != a.rank) {
    __threadfence_system();  // earlier writes of this GPU (previous kernels of the stream) precede the signal
    uint32_t* remote = a.flags[t] + a.channel * 8 + a.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(a.epoch) : "memory");
    const uint32_t* mine = a.flags[a.rank] + a.channel * 8 + t;
    const long long t0 = clock64();
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int32_t>(v - a.epoch) >= 0) break;
      if (clock64() - t0 > a.limit) {  // bounded: record which wait gave up and return
        if (a.status != nullptr) atomicCAS(a.status, 0, LEANFFN_DEV_TIMEOUT_PEER);
        break;
      }
      __nanosleep(64);
    }
  }
}

int32_t launch_peer_barrier(void* const* flags, int32_t rank, int32_t world, int32_t channel, uint32_t epoch,
                            long long limit, int32_t* status, cudaStream_t st) {
  PeerBarrierArgs a{};
  for (int i = 0; i < world; ++i) a.flags[i] = static_cast<uint32_t*>(flags[i]);
  a.rank = rank, a.world = world, a.channel = channel, a.epoch = epoch, a.limit = limit, a.status = status;
  peer_barrier_kernel<<<1, 32, 0, st>>>(a);
  return launch_status();
}

// ---- split of fp32 values into two TF32-exact parts -------------------------------------------------
// hi = x with the 13 low mantissa bits cleared (what a TF32 multiplication reads), lo = x - hi (exact in fp32).
// Per slice the A operand is laid out as (hi | lo | hi) and the B operand as (lo | hi | hi).
__global__ void split_tf32_kernel(const float* __restrict__ x, int64_t ldx, float* __restrict__ out, int64_t rows,
                                  int64_t cols, int role, int64_t slice) {
  const int64_t total = rows * cols;
  const int64_t slices = cols / slice > 0 ? cols / slice : 1;  // the last slice takes the remainder
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    int64_t s = c / slice;
    if (s >= slices) s = slices - 1;
    const int64_t first = s * slice;
    const int64_t width = s == slices - 1 ? cols - first : slice;
    const float v = x[r * ldx + c];
    const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    const float lo = v - hi;
    // parts of a slice: (a_hi b_lo) and (a_lo b_hi) come first, (a_hi b_hi) last.  The small cross terms then add up
    // while the accumulator is still tiny (its truncation steps are 2^-11 of the result's), and only the last third
    // of the slice's instructions truncate an accumulator of full size.
    float* o = out + r * 3 * cols + 3 * first + (c - first);
    o[0] = role == 0 ? hi : lo;
    o[width] = role == 0 ? lo : hi;
    o[2 * width] = hi;
  }
}

cudaError_t launch_split_tf32(const float* x, int64_t ldx, float* out, int64_t rows, int64_t cols, int role,
                              int64_t slice, cudaStream_t st) {
  const int64_t total = rows * cols;
  const int64_t want = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  split_tf32_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, st>>>(x, ldx, out, rows, cols, role,
                                                                                slice);
  return cudaGetLastError();
}

}  // namespace leanffn

using namespace leanffn;

// ---- C ABI -------------------------------------------------------------------------------------
#define DT2(a, b) ((a) * 2 + (b))
static inline bool dtype_ok(int32_t d) { return d == LEANFFN_F32 || d == LEANFFN_BF16; }

extern "C" int32_t leanffn_layer_norm_forward(const void* x, int32_t x_dtype, const void* gamma, const void* beta,
                                              int32_t param_dtype, void* y, int32_t y_dtype, int64_t rows,
                                              int64_t cols, float eps, float dropout_p, uint64_t seed,
                                              uint64_t elem_offset, const void* residual, int32_t residual_dtype,
                                              void* stream) {
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff) return LEANFFN_ERR_SHAPE;
  if (rows > 0 && (x == nullptr || y == nullptr)) return LEANFFN_ERR_NULL;
  if (!dtype_ok(x_dtype) || !dtype_ok(param_dtype) || !dtype_ok(y_dtype)) return LEANFFN_ERR_DTYPE;
  if (residual != nullptr && !dtype_ok(residual_dtype)) return LEANFFN_ERR_DTYPE;
  if (!(dropout_p >= 0.f && dropout_p < 1.f)) return LEANFFN_ERR_UNSUPPORTED;
  if (rows == 0) return LEANFFN_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint32_t thr = dropout_p > 0.f ? dropout_threshold(dropout_p) : 0u;
  const float ks = 1.0f / (1.0f - dropout_p);
  if (residual == nullptr) residual_dtype = x_dtype;
  // Supported (x, param, y, residual) element types: the combinations the fp32 path, the bf16 path
  // with an fp32 residual stream, and the all-bf16 path produce. Anything else is rejected.
#define LN_FWD_GO(TX, TP, TY, TR) \
  return ln_fwd_dispatch<TX, TP, TY, TR>(x, gamma, beta, y, residual, rows, cols, eps, thr, ks, seed, elem_offset, st)
  const int key = x_dtype * 8 + param_dtype * 4 + y_dtype * 2 + residual_dtype;
  switch (key) {
    case 0: LN_FWD_GO(float, float, float, float);
    case 2: LN_FWD_GO(float, float, bf16, float);
    case 10: LN_FWD_GO(bf16, float, bf16, float);
    case 11: LN_FWD_GO(bf16, float, bf16, bf16);
    case 15: LN_FWD_GO(bf16, bf16, bf16, bf16);
    default: return LEANFFN_ERR_DTYPE;
  }
#undef LN_FWD_GO
}

extern "C" size_t leanffn_layer_norm_backward_scratch_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  const LnBwdPlan plan = ln_bwd_plan(rows, cols);
  const int64_t chunks = colsum_chunks(plan.part_rows, 2 * cols);
  return sizeof(float) * static_cast<size_t>(plan.part_rows * 2 * cols + 2 * cols + chunks * 2 * cols);
}

extern "C" int32_t leanffn_layer_norm_backward(const void* dy, int32_t dy_dtype, const void* x, int32_t x_dtype,
                                               const void* gamma, int32_t param_dtype, const void* dresidual,
                                               int32_t dresidual_dtype, void* dx, int32_t dx_dtype, float* dgamma,
                                               float* dbeta, void* scratch, int64_t rows, int64_t cols, float eps,
                                               void* stream) {
  if (dy == nullptr || x == nullptr) return LEANFFN_ERR_NULL;
  if ((dgamma == nullptr) != (dbeta == nullptr)) return LEANFFN_ERR_NULL;
  if (dgamma != nullptr && scratch == nullptr) return LEANFFN_ERR_NULL;
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff) return LEANFFN_ERR_SHAPE;
  if (!dtype_ok(dy_dtype) || !dtype_ok(x_dtype) || !dtype_ok(param_dtype) || !dtype_ok(dx_dtype))
    return LEANFFN_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    if (dgamma != nullptr) {
      cudaMemsetAsync(dgamma, 0, sizeof(float) * cols, st);
      cudaMemsetAsync(dbeta, 0, sizeof(float) * cols, st);
    }
    return LEANFFN_OK;
  }
  if (cols % 4 == 0 && cols <= 16384) {
    // the register path moves 4-element vectors
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al16(dy) || !al16(x) || !al16(gamma) || !al16(dresidual) || !al16(dx) || !al16(scratch)) return LEANFFN_ERR_ALIGN;
  }
  if (dresidual == nullptr) dresidual_dtype = dy_dtype;
#define LN_BWD_GO(TD, TX, TP, TR, TO)                                                                             \
  return ln_bwd_dispatch<TD, TX, TP, TR, TO>(dy, x, gamma, dresidual, dx, dgamma, dbeta, scratch, rows, cols, eps, \
                                             st)
  // Supported (dy, x, param, dresidual, dx) element types; see leanffn_layer_norm_forward.
  const int key = dy_dtype * 16 + x_dtype * 8 + param_dtype * 4 + dresidual_dtype * 2 + dx_dtype;
  switch (key) {
    case 0: LN_BWD_GO(float, float, float, float, float);
    case 18: LN_BWD_GO(bf16, float, float, bf16, float);
    case 27: LN_BWD_GO(bf16, bf16, float, bf16, bf16);
    case 31: LN_BWD_GO(bf16, bf16, bf16, bf16, bf16);
    default: return LEANFFN_ERR_DTYPE;
  }
#undef LN_BWD_GO
}

namespace leanffn {
// Launchers shared with the GEMM entry point (SIMT path applies the activation as a second pass).
int32_t launch_act_fwd(const void* pre, void* hid, int32_t dtype, int64_t rows, int64_t inter, int32_t gated,
                       int32_t act, cudaStream_t st) {
  const int grid = grid_for(rows * (inter / 4), 256);
  if (dtype == LEANFFN_BF16)
    act_fwd_kernel<bf16, true><<<grid, 256, 0, st>>>(static_cast<const bf16*>(pre), static_cast<bf16*>(hid), rows,
                                                     inter, gated, act);
  else
    act_fwd_kernel<float, false><<<grid, 256, 0, st>>>(static_cast<const float*>(pre), static_cast<float*>(hid), rows,
                                                       inter, gated, act);
  return launch_status();
}
// dhid may alias the linear half of dpre (row pitch ld_dhid): every thread reads its elements before
// it overwrites them.
int32_t launch_act_bwd(const void* dhid, int64_t ld_dhid, const void* pre, void* dpre, void* hid_out, int32_t dtype,
                       int64_t rows, int64_t inter, int32_t gated, int32_t act, cudaStream_t st) {
  const int grid = grid_for(rows * (inter / 4), 256);
  if (dtype == LEANFFN_BF16)
    act_bwd_kernel<bf16, true><<<grid, 256, 0, st>>>(static_cast<const bf16*>(dhid), ld_dhid,
                                                     static_cast<const bf16*>(pre), static_cast<bf16*>(dpre),
                                                     static_cast<bf16*>(hid_out), rows, inter, gated, act);
  else
    act_bwd_kernel<float, false><<<grid, 256, 0, st>>>(static_cast<const float*>(dhid), ld_dhid,
                                                       static_cast<const float*>(pre), static_cast<float*>(dpre),
                                                       static_cast<float*>(hid_out), rows, inter, gated, act);
  return launch_status();
}
}  // namespace leanffn

extern "C" int32_t leanffn_activation_forward(const void* pre, void* hid, int32_t dtype, int64_t rows, int64_t inter,
                                              int32_t gated, int32_t act, void* stream) {
  if (pre == nullptr || hid == nullptr) return LEANFFN_ERR_NULL;
  if (rows < 0 || inter <= 0 || inter % 4 != 0) return LEANFFN_ERR_SHAPE;
  if (!dtype_ok(dtype)) return LEANFFN_ERR_DTYPE;
  if (act < 0 || act >= LEANFFN_ACT_COUNT) return LEANFFN_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(pre) | reinterpret_cast<uintptr_t>(hid)) & 15u) return LEANFFN_ERR_ALIGN;
  if (rows == 0) return LEANFFN_OK;
  return launch_act_fwd(pre, hid, dtype, rows, inter, gated, act, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t leanffn_activation_backward(const void* dhid, const void* pre, void* dpre, void* hid_out,
                                               int32_t dtype, int64_t rows, int64_t inter, int32_t gated, int32_t act,
                                               void* stream) {
  if (dhid == nullptr || pre == nullptr || dpre == nullptr) return LEANFFN_ERR_NULL;
  if (rows < 0 || inter <= 0 || inter % 4 != 0) return LEANFFN_ERR_SHAPE;
  if (!dtype_ok(dtype)) return LEANFFN_ERR_DTYPE;
  if (act < 0 || act >= LEANFFN_ACT_COUNT) return LEANFFN_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(dhid) | reinterpret_cast<uintptr_t>(pre) | reinterpret_cast<uintptr_t>(dpre) |
       reinterpret_cast<uintptr_t>(hid_out)) & 15u)
    return LEANFFN_ERR_ALIGN;
  if (rows == 0) return LEANFFN_OK;
  return launch_act_bwd(dhid, inter, pre, dpre, hid_out, dtype, rows, inter, gated, act,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int32_t leanffn_dropout(const void* x, int32_t x_dtype, void* y, int32_t y_dtype, int64_t n, float p,
                                   uint64_t seed, uint64_t elem_offset, const void* residual, int32_t residual_dtype,
                                   void* stream) {
  if (x == nullptr || y == nullptr) return LEANFFN_ERR_NULL;
  if (n < 0) return LEANFFN_ERR_SHAPE;
  if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return LEANFFN_ERR_DTYPE;
  if (residual != nullptr && !dtype_ok(residual_dtype)) return LEANFFN_ERR_DTYPE;
  if (!(p >= 0.f && p < 1.f)) return LEANFFN_ERR_UNSUPPORTED;
  if (n == 0) return LEANFFN_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint32_t thr = p > 0.f ? dropout_threshold(p) : 0u;
  const float ks = 1.0f / (1.0f - p);
  const int vec_ok = (elem_offset % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(y) % 16 == 0) && (reinterpret_cast<uintptr_t>(residual) % 16 == 0);
  const int grid = grid_for((n + 3) / 4, 256);
  if (residual == nullptr) residual_dtype = LEANFFN_F32;
#define DROP_GO(TX, TY, TR)                                                                                  \
  dropout_kernel<TX, TY, TR><<<grid, 256, 0, st>>>(static_cast<const TX*>(x), static_cast<TY*>(y),           \
                                                   static_cast<const TR*>(residual), n, thr, ks, seed,       \
                                                   elem_offset, vec_ok)
  switch (x_dtype * 4 + y_dtype * 2 + residual_dtype) {
    case 0: DROP_GO(float, float, float); break;
    case 1: DROP_GO(float, float, bf16); break;
    case 2: DROP_GO(float, bf16, float); break;
    case 3: DROP_GO(float, bf16, bf16); break;
    case 4: DROP_GO(bf16, float, float); break;
    case 5: DROP_GO(bf16, float, bf16); break;
    case 6: DROP_GO(bf16, bf16, float); break;
    default: DROP_GO(bf16, bf16, bf16); break;
  }
#undef DROP_GO
  return launch_status();
}

extern "C" int32_t leanffn_dropout_mask(uint8_t* mask, int64_t n, float p, uint64_t seed, uint64_t elem_offset,
                                        void* stream) {
  if (mask == nullptr) return LEANFFN_ERR_NULL;
  if (n < 0) return LEANFFN_ERR_SHAPE;
  if (!(p >= 0.f && p < 1.f)) return LEANFFN_ERR_UNSUPPORTED;
  if (n == 0) return LEANFFN_OK;
  dropout_mask_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      mask, n, p > 0.f ? dropout_threshold(p) : 0u, seed, elem_offset);
  return launch_status();
}

extern "C" size_t leanffn_column_sum_scratch_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return sizeof(float) * static_cast<size_t>(colsum_chunks(rows, cols) * cols);
}

extern "C" int32_t leanffn_column_sum(const void* x, int32_t x_dtype, int64_t ld, float* out, void* scratch,
                                      int64_t rows, int64_t cols, void* stream) {
  if (x == nullptr || out == nullptr) return LEANFFN_ERR_NULL;
  if (rows < 0 || cols <= 0 || ld < cols) return LEANFFN_ERR_SHAPE;
  if (!dtype_ok(x_dtype)) return LEANFFN_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    cudaMemsetAsync(out, 0, sizeof(float) * cols, st);
    return launch_status();
  }
  if (colsum_chunks(rows, cols) > 1 && scratch == nullptr) return LEANFFN_ERR_NULL;
  if (x_dtype == LEANFFN_BF16)
    return colsum_launch<bf16>(static_cast<const bf16*>(x), ld, out, static_cast<float*>(scratch), rows, cols, st);
  return colsum_launch<float>(static_cast<const float*>(x), ld, out, static_cast<float*>(scratch), rows, cols, st);
}

extern "C" size_t leanffn_dropout_colsum_scratch_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  const int64_t fused = dropout_colsum_chunks(rows, cols);
  // fused path: [chunks, cols] partials + the second stage's own scratch; unfused path: the plain column sum's scratch
  const int64_t a = fused * cols + colsum_chunks(fused, cols) * cols;
  const int64_t b = colsum_chunks(rows, cols) * cols;
  return sizeof(float) * static_cast<size_t>(a > b ? a : b);
}

extern "C" int32_t leanffn_dropout_colsum(const void* x, int32_t x_dtype, void* y, int32_t y_dtype, int64_t rows,
                                          int64_t cols, float p, uint64_t seed, uint64_t elem_offset, float* colsum,
                                          void* scratch, void* stream) {
  if (x == nullptr || y == nullptr || colsum == nullptr) return LEANFFN_ERR_NULL;
  if (rows < 0 || cols <= 0) return LEANFFN_ERR_SHAPE;
  if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return LEANFFN_ERR_DTYPE;
  if (!(p >= 0.f && p < 1.f)) return LEANFFN_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    cudaMemsetAsync(colsum, 0, sizeof(float) * cols, st);
    return launch_status();
  }
  if (scratch == nullptr) return LEANFFN_ERR_NULL;
  const bool fused = cols % 8 == 0 && elem_offset % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(y) % 16 == 0 && reinterpret_cast<uintptr_t>(scratch) % 16 == 0;
  if (!fused) {
    const int32_t s = leanffn_dropout(x, x_dtype, y, y_dtype, rows * cols, p, seed, elem_offset, nullptr, 0, stream);
    if (s != LEANFFN_OK) return s;
    return leanffn_column_sum(y, y_dtype, cols, colsum, scratch, rows, cols, stream);
  }
  const uint32_t thr = p > 0.f ? dropout_threshold(p) : 0u;
  const float ks = 1.0f / (1.0f - p);
  const int64_t chunks = dropout_colsum_chunks(rows, cols);
  const int64_t rpc = (rows + chunks - 1) / chunks;
  float* partial = static_cast<float*>(scratch);
  const dim3 grid(static_cast<unsigned>((cols + 255) / 256), static_cast<unsigned>(chunks));
#define DC_GO(TX, TY)                                                                                              \
  dropout_colsum_kernel<TX, TY><<<grid, 256, 0, st>>>(static_cast<const TX*>(x), static_cast<TY*>(y), partial, rows, \
                                                      cols, rpc, thr, ks, seed, elem_offset)
  switch (x_dtype * 2 + y_dtype) {
    case 0: DC_GO(float, float); break;
    case 1: DC_GO(float, bf16); break;
    case 2: DC_GO(bf16, float); break;
    default: DC_GO(bf16, bf16); break;
  }
#undef DC_GO
  const int32_t s = launch_status();
  if (s != LEANFFN_OK) return s;
  return colsum_launch<float>(partial, cols, colsum, partial + chunks * cols, chunks, cols, st);
}

// ---- column sum without any allocation --------------------------------------------------------------------
// Scratch for leanffn_column_sum_static lives in the library image: 1 MiB per GPU that loads the library, held
// until the process exits.  In host code the array's name is only a handle; the device address is looked up once
// per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
constexpr int64_t STATIC_SCRATCH_FLOATS = 1 << 18;
constexpr int64_t STATIC_MAX_COLS = 65536;
static __device__ __align__(256) float g_colsum_static_scratch[STATIC_SCRATCH_FLOATS];
static float* g_colsum_static_ptr[64] = {nullptr};

extern "C" int64_t leanffn_column_sum_static_capacity(void) { return STATIC_SCRATCH_FLOATS; }

extern "C" int32_t leanffn_column_sum_static(const void* x, int32_t x_dtype, int64_t ld, float* out, int64_t rows,
                                             int64_t cols, void* stream) {
  if (rows < 0 || cols <= 0 || ld < cols) return LEANFFN_ERR_SHAPE;
  if (out == nullptr || (rows > 0 && x == nullptr)) return LEANFFN_ERR_NULL;
  if (!dtype_ok(x_dtype)) return LEANFFN_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    cudaMemsetAsync(out, 0, sizeof(float) * cols, st);
    return launch_status();
  }
  if (cols > STATIC_MAX_COLS) return LEANFFN_ERR_TOO_LARGE;
  const int64_t chunks = colsum_chunks(rows, cols);
  if (chunks > 1 && chunks * cols > STATIC_SCRATCH_FLOATS) return LEANFFN_ERR_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return 1000 + static_cast<int32_t>(e);
  if (dev < 0 || dev >= 64) return LEANFFN_ERR_UNSUPPORTED;
  if (g_colsum_static_ptr[dev] == nullptr) {
    // first call on this device (it is the current device): resolve the symbol's device address
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_colsum_static_scratch);
    if (e != cudaSuccess) return 1000 + static_cast<int32_t>(e);
    if (ptr == nullptr) return LEANFFN_ERR_DRIVER;
    g_colsum_static_ptr[dev] = ptr;
  }
  float* scratch = g_colsum_static_ptr[dev];
  // Every partial the second stage reads is written by the first stage of the same call, so nothing left in
  // the array by an earlier call is ever consumed and nothing needs clearing.
  if (x_dtype == LEANFFN_BF16)
    return colsum_launch<bf16>(static_cast<const bf16*>(x), ld, out, scratch, rows, cols, st);
  return colsum_launch<float>(static_cast<const float*>(x), ld, out, scratch, rows, cols, st);
}

extern "C" int32_t leanffn_cast(const void* x, int32_t x_dtype, void* y, int32_t y_dtype, int64_t n, void* stream) {
  return leanffn_dropout(x, x_dtype, y, y_dtype, n, 0.f, 0, 0, nullptr, 0, stream);
}

extern "C" int32_t leanffn_transpose(const void* x, int32_t dtype, int64_t ldx, void* y, int64_t rows, int64_t cols,
                                     void* stream) {
  if (x == nullptr || y == nullptr) return LEANFFN_ERR_NULL;
  if (rows < 0 || cols < 0 || ldx < cols) return LEANFFN_ERR_SHAPE;
  if (!dtype_ok(dtype)) return LEANFFN_ERR_DTYPE;
  if (rows == 0 || cols == 0) return LEANFFN_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>((cols + 63) / 64), static_cast<unsigned>((rows + 63) / 64));
  if (dtype == LEANFFN_BF16)
    transpose_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, static_cast<bf16*>(y), rows, cols);
  else
    transpose_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), ldx, static_cast<float*>(y), rows,
                                                  cols);
  return launch_status();
}
