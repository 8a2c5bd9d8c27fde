// SIMT (CUDA-core) GEMM with fp32 accumulation.  It is the fp32-mode product kernel (plain TF32 would
// miss the 1e-4 parity bound), the path for shapes the tensor-core kernel rejects (block sizes that
// are not multiples of 128, rows whose pitch is not a multiple of 16 bytes), and an on-device
// cross-check for the tcgen05 kernels.  Operands are addressed through (m,k) / (n,k) strides so every
// majorness and all three block-sparse products share one kernel.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gemm_common.cuh"

namespace leanffn {

constexpr int SB_M = 64, SB_N = 64, SB_K = 16, S_THREADS = 256;

// Block-sparse addressing.  The table holds int32 pairs:
//   forward (MODE 1): row = output block, entry t = (weight block f, input block j)
//   dgrad   (MODE 2): row = input block,  entry t = (weight block f, output block o)
//   wgrad   (MODE 3): row = weight block f, single entry (output block o, input block j)
// Weight block f is a [block(out) x block(in)] row-major matrix at B + f * block * block.
// kk runs over the compressed reduction axis (entries * block for forward / dgrad, tokens for wgrad).
__device__ __forceinline__ int2 bs_entry(const SimtOperands& o, int64_t row, int64_t t) {
  return __ldg(reinterpret_cast<const int2*>(o.bs_index) + row * o.bs_nnz + t);
}
__device__ __forceinline__ int bs_row_count(const SimtOperands& o, int64_t row) {
  return o.bs_count != nullptr ? __ldg(o.bs_count + row) : o.bs_nnz;
}
template <int MODE>
__device__ __forceinline__ void bs_addr(const SimtOperands& o, int64_t m, int64_t n, int64_t kk, int64_t& ia,
                                        int64_t& ib) {
  const int bs = o.bs_block;
  if constexpr (MODE == 1) {
    const int2 e = bs_entry(o, n / bs, kk / bs);
    ia = m * o.lda + static_cast<int64_t>(e.y) * bs + kk % bs;
    ib = (static_cast<int64_t>(e.x) * bs + n % bs) * bs + kk % bs;
  } else if constexpr (MODE == 2) {
    const int2 e = bs_entry(o, n / bs, kk / bs);
    ia = m * o.lda + static_cast<int64_t>(e.y) * bs + kk % bs;
    ib = (static_cast<int64_t>(e.x) * bs + kk % bs) * bs + n % bs;
  } else {
    const int2 e = bs_entry(o, m / bs, 0);
    ia = kk * o.lda + static_cast<int64_t>(e.x) * bs + m % bs;
    ib = kk * o.ldb + static_cast<int64_t>(e.y) * bs + n;
  }
}

template <typename TIN, int MODE>
__global__ void __launch_bounds__(S_THREADS)
gemm_simt_kernel(SimtOperands o, EpiParams ep) {
  __shared__ float As[SB_K][SB_M + 4];
  __shared__ float Bs[SB_K][SB_N + 4];
  const int tid = threadIdx.x;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * SB_M, n0 = static_cast<int64_t>(blockIdx.x) * SB_N;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int pass = 0; pass < 2; ++pass) {
    const TIN* A = static_cast<const TIN*>(pass == 0 ? o.A : o.A2);
    const TIN* B = static_cast<const TIN*>(pass == 0 ? o.B : o.B2);
    int K = pass == 0 ? o.K : o.K2;
    if (MODE == 1 || MODE == 2) {
      if (pass == 0) K = bs_row_count(o, n0 / o.bs_block) * o.bs_block;
    }
    if (K <= 0 || A == nullptr) continue;
    const int64_t a_sm = pass == 0 ? o.a_sm : o.a2_sm, a_sk = pass == 0 ? o.a_sk : o.a2_sk;
    const int64_t b_sn = pass == 0 ? o.b_sn : o.b2_sn, b_sk = pass == 0 ? o.b_sk : o.b2_sk;
    const bool sparse = (MODE != 0) && pass == 0;
    const bool a_kfast = sparse ? (MODE != 3) : (a_sk == 1);
    const bool b_kfast = sparse ? (MODE == 1) : (b_sk == 1);
    for (int k0 = 0; k0 < K; k0 += SB_K) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = tid + i * S_THREADS;
        {
          const int kk = a_kfast ? (e % SB_K) : (e / SB_M);
          const int mm = a_kfast ? (e / SB_K) : (e % SB_M);
          const int64_t m = m0 + mm, k = k0 + kk;
          float v = 0.f;
          if (m < ep.M && k < K) {
            if (sparse) {
              // the tile's first column / row names the block: tiles never straddle blocks here
              // (block % 64 == 0; smaller blocks use the per-element kernel below)
              int64_t ia, ib;
              bs_addr<MODE == 0 ? 1 : MODE>(o, m, n0, k, ia, ib);
              v = to_f32(A[ia]);
            } else {
              v = to_f32(A[m * a_sm + k * a_sk]);
            }
          }
          As[kk][mm] = v;
        }
        {
          const int kk = b_kfast ? (e % SB_K) : (e / SB_N);
          const int nn = b_kfast ? (e / SB_K) : (e % SB_N);
          const int64_t n = n0 + nn, k = k0 + kk;
          float v = 0.f;
          if (n < ep.N && k < K) {
            if (sparse) {
              int64_t ia, ib;
              bs_addr<MODE == 0 ? 1 : MODE>(o, m0, n, k, ia, ib);
              v = to_f32(B[ib]);
            } else
              v = to_f32(B[n * b_sn + k * b_sk]);
          }
          Bs[kk][nn] = v;
        }
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < SB_K; ++kk) {
        const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
        const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= ep.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n < ep.N) epilogue_scalar(ep, m, n, acc[i][j]);
    }
  }
}

// Block-sparse products whose block is smaller than the tile: one thread per output element, the
// reduction walked block by block.  Only small test layouts (block 8 / 16 / 32) come here.
template <typename TIN, int MODE>
__global__ void __launch_bounds__(256)
gemm_simt_smallblock_kernel(SimtOperands o, EpiParams ep) {
  const TIN* A = static_cast<const TIN*>(o.A);
  const TIN* B = static_cast<const TIN*>(o.B);
  const int64_t total = static_cast<int64_t>(ep.M) * ep.N;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = e / ep.N, n = e - m * ep.N;
    float acc = 0.f;
    const int64_t K = (MODE == 3) ? o.K : static_cast<int64_t>(bs_row_count(o, n / o.bs_block)) * o.bs_block;
    for (int64_t k = 0; k < K; ++k) {
      int64_t ia, ib;
      bs_addr<MODE>(o, m, n, k, ia, ib);
      acc = fmaf(to_f32(A[ia]), to_f32(B[ib]), acc);
    }
    if (o.K2 > 0 && o.A2 != nullptr) {
      const TIN* A2 = static_cast<const TIN*>(o.A2);
      const TIN* B2 = static_cast<const TIN*>(o.B2);
      for (int64_t k = 0; k < o.K2; ++k)
        acc = fmaf(to_f32(A2[m * o.a2_sm + k * o.a2_sk]), to_f32(B2[n * o.b2_sn + k * o.b2_sk]), acc);
    }
    epilogue_scalar(ep, m, n, acc);
  }
}

template <typename TIN>
static cudaError_t simt_launch(const SimtOperands& o, const EpiParams& ep, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((ep.N + SB_N - 1) / SB_N), static_cast<unsigned>((ep.M + SB_M - 1) / SB_M));
  const bool small = o.bs_mode != 0 && (o.bs_block % SB_N != 0);
  if (small) {
    const int64_t total = static_cast<int64_t>(ep.M) * ep.N;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const unsigned g = static_cast<unsigned>(blocks);
    switch (o.bs_mode) {
      case 1: gemm_simt_smallblock_kernel<TIN, 1><<<g, 256, 0, st>>>(o, ep); break;
      case 2: gemm_simt_smallblock_kernel<TIN, 2><<<g, 256, 0, st>>>(o, ep); break;
      default: gemm_simt_smallblock_kernel<TIN, 3><<<g, 256, 0, st>>>(o, ep); break;
    }
    return cudaGetLastError();
  }
  switch (o.bs_mode) {
    case 0: gemm_simt_kernel<TIN, 0><<<grid, S_THREADS, 0, st>>>(o, ep); break;
    case 1: gemm_simt_kernel<TIN, 1><<<grid, S_THREADS, 0, st>>>(o, ep); break;
    case 2: gemm_simt_kernel<TIN, 2><<<grid, S_THREADS, 0, st>>>(o, ep); break;
    default: gemm_simt_kernel<TIN, 3><<<grid, S_THREADS, 0, st>>>(o, ep); break;
  }
  return cudaGetLastError();
}

cudaError_t gemm_simt(const SimtOperands& o, const EpiParams& ep, int32_t in_dtype, cudaStream_t st) {
  if (in_dtype == LEANFFN_BF16) return simt_launch<bf16>(o, ep, st);
  return simt_launch<float>(o, ep, st);
}

}  // namespace leanffn
