// Element conversions, activation functions with their derivatives, and the counter-based
// Philox4x32-10 keep-mask shared by every kernel that applies dropout.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/leanffn_b200.h"

namespace leanffn {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float v) {
  return __float2bfloat16_rn(v);
}

// 4-element vectors (16 bytes of fp32, 8 bytes of bf16).
template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  float4 raw;
  __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
  __device__ __forceinline__ void get(float (&f)[4]) const {
    f[0] = raw.x, f[1] = raw.y, f[2] = raw.z, f[3] = raw.w;
  }
  __device__ __forceinline__ void set(const float (&f)[4]) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <>
struct Vec4<bf16> {
  uint2 raw;
  __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint2*>(p) = raw; }
  __device__ __forceinline__ void get(float (&f)[4]) const {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    f[0] = __low2float(a), f[1] = __high2float(a), f[2] = __low2float(b), f[3] = __high2float(b);
  }
  __device__ __forceinline__ void set(const float (&f)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(f[2], f[3]);
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
  }
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ---- activations ------------------------------------------------------------------------------
// FAST selects hardware approximations (tanh.approx / __expf); their error is below one bf16 ulp,
// so the bf16 kernels use them and the fp32 kernels do not.
template <bool FAST>
__device__ __forceinline__ float tanh_f(float x) {
  if constexpr (FAST) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  } else {
    return tanhf(x);
  }
}
template <bool FAST>
__device__ __forceinline__ float sigmoid_f(float x) {
  if constexpr (FAST) {
    return __fdividef(1.0f, 1.0f + __expf(-x));
  } else {
    return 1.0f / (1.0f + expf(-x));
  }
}

// gelu_fused and its derivative (lean_transformer/utils.py:24-38) with the common subexpressions shared and every
// multiply-add written as one fused operation: 10 arithmetic instructions and one tanh for both values.
//   u = 0.79788456 x (1 + 0.044715 x^2),  t = tanh(u),  y = 0.5 x (1 + t),
//   d = 0.5 x (1 - t^2) (0.79788456 + 0.1070322243 x^2) + 0.5 (1 + t)
template <bool FAST>
__device__ __forceinline__ float gelu_tanh_fwd(float x) {
  const float xx = x * x;
  const float t = tanh_f<FAST>(x * fmaf(xx, 0.79788456f * 0.044715f, 0.79788456f));
  const float h = 0.5f * x;
  return fmaf(h, t, h);
}
template <bool FAST>
__device__ __forceinline__ void gelu_tanh_fwd_bwd(float x, float& y, float& d) {
  const float xx = x * x;
  const float t = tanh_f<FAST>(x * fmaf(xx, 0.79788456f * 0.044715f, 0.79788456f));
  const float h = 0.5f * x;
  y = fmaf(h, t, h);
  const float one_minus_tt = fmaf(-t, t, 1.0f);
  const float q = fmaf(xx, 0.1070322243f, 0.79788456f);
  d = fmaf(h * one_minus_tt, q, fmaf(0.5f, t, 0.5f));
}

// y = act(x); d = act'(x)
template <bool FAST>
__device__ __forceinline__ void act_fwd_bwd(int act, float x, float& y, float& d) {
  switch (act) {
    case LEANFFN_ACT_GELU_TANH:
      gelu_tanh_fwd_bwd<FAST>(x, y, d);
      break;
    case LEANFFN_ACT_GELU_ERF: {
      const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
      y = x * cdf;
      d = cdf + x * 0.39894228040143268f * expf(-0.5f * x * x);
      break;
    }
    case LEANFFN_ACT_RELU:
      y = x > 0.0f ? x : 0.0f;
      d = x > 0.0f ? 1.0f : 0.0f;
      break;
    case LEANFFN_ACT_SILU: {
      const float s = sigmoid_f<FAST>(x);
      y = x * s;
      d = s * (1.0f + x * (1.0f - s));
      break;
    }
    case LEANFFN_ACT_TANH: {
      const float t = tanh_f<FAST>(x);
      y = t;
      d = 1.0f - t * t;
      break;
    }
    case LEANFFN_ACT_SIGMOID: {
      const float s = sigmoid_f<FAST>(x);
      y = s;
      d = s * (1.0f - s);
      break;
    }
    default:
      y = x;
      d = 1.0f;
      break;
  }
}
template <bool FAST>
__device__ __forceinline__ float act_fwd(int act, float x) {
  switch (act) {
    case LEANFFN_ACT_GELU_TANH:
      return gelu_tanh_fwd<FAST>(x);
    case LEANFFN_ACT_GELU_ERF:
      return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    case LEANFFN_ACT_RELU:
      return x > 0.0f ? x : 0.0f;
    case LEANFFN_ACT_SILU:
      return x * sigmoid_f<FAST>(x);
    case LEANFFN_ACT_TANH:
      return tanh_f<FAST>(x);
    case LEANFFN_ACT_SIGMOID:
      return sigmoid_f<FAST>(x);
    default:
      return x;
  }
}

// Compile-time selected variants for the GEMM epilogues: ACT >= 0 inlines exactly one activation (small code, the
// hot loops stay in the instruction cache); ACT < 0 falls back to the run-time switch.
template <int ACT, bool FAST>
__device__ __forceinline__ float act_fwd_t(int act, float x) {
  if constexpr (ACT == LEANFFN_ACT_GELU_TANH) {
    return gelu_tanh_fwd<FAST>(x);
  } else if constexpr (ACT == LEANFFN_ACT_SILU) {
    return x * sigmoid_f<FAST>(x);
  } else if constexpr (ACT == LEANFFN_ACT_RELU) {
    return x > 0.0f ? x : 0.0f;
  } else {
    return act_fwd<FAST>(act, x);
  }
}
template <int ACT, bool FAST>
__device__ __forceinline__ void act_fwd_bwd_t(int act, float x, float& y, float& d) {
  if constexpr (ACT == LEANFFN_ACT_GELU_TANH) {
    gelu_tanh_fwd_bwd<FAST>(x, y, d);
  } else if constexpr (ACT == LEANFFN_ACT_SILU) {
    const float s = sigmoid_f<FAST>(x);
    y = x * s;
    d = s * (1.0f + x * (1.0f - s));
  } else if constexpr (ACT == LEANFFN_ACT_RELU) {
    y = x > 0.0f ? x : 0.0f;
    d = x > 0.0f ? 1.0f : 0.0f;
  } else {
    act_fwd_bwd<FAST>(act, x, y, d);
  }
}

// ---- Philox4x32-10 ----------------------------------------------------------------------------
// Counter (g lo, g hi, 0, 0) with g = element_index >> 2, key (seed lo, seed hi); element e uses
// output word e & 3.
__device__ __forceinline__ uint4 philox4x32_10(uint64_t group, uint64_t seed) {
  uint32_t c0 = static_cast<uint32_t>(group), c1 = static_cast<uint32_t>(group >> 32), c2 = 0u, c3 = 0u;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0, c1 = lo1, c2 = n2, c3 = lo0;
    k0 += 0x9E3779B9u, k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}
__host__ __device__ __forceinline__ uint32_t dropout_threshold(float p) {
  const double t = static_cast<double>(p) * 4294967296.0;
  return t >= 4294967295.0 ? 0xFFFFFFFFu : static_cast<uint32_t>(t);
}
// keep flags for the aligned group of 4 elements starting at element index 4*group
__device__ __forceinline__ void dropout_keep4(uint64_t group, uint64_t seed, uint32_t threshold, bool (&keep)[4]) {
  const uint4 r = philox4x32_10(group, seed);
  keep[0] = r.x >= threshold, keep[1] = r.y >= threshold, keep[2] = r.z >= threshold, keep[3] = r.w >= threshold;
}
__device__ __forceinline__ bool dropout_keep1(uint64_t elem, uint64_t seed, uint32_t threshold) {
  const uint4 r = philox4x32_10(elem >> 2, seed);
  const uint32_t w = (elem & 3) == 0 ? r.x : (elem & 3) == 1 ? r.y : (elem & 3) == 2 ? r.z : r.w;
  return w >= threshold;
}

}  // namespace leanffn
