// Row arithmetic shared by the bulk-copy AdaLN / AdaRMSNorm kernels: conversion of a 16-byte
// vector to packed fp32 pairs (the math then runs on the packed fp32 pipe of sm_100: add / mul /
// fma on two floats per instruction), the CTA-wide row reduction, and the reciprocal square root.
#pragma once

#include "norm_impl.cuh"

namespace nd {

template <typename T, int VEC>
__device__ __forceinline__ void unpack2(const Vec<T, VEC>& v, float2 (&f)[VEC / 2]) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(v.v);
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      f[i].x = __uint_as_float(w[i] << 16);
      f[i].y = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else if constexpr (std::is_same<T, __half>::value) {
    const __half2* h = reinterpret_cast<const __half2*>(v.v);
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) f[i] = __half22float2(h[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) f[i] = make_float2(v.v[2 * i], v.v[2 * i + 1]);
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void pack2(const float2 (&f)[VEC / 2], Vec<T, VEC>& v) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(v.v);
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) o[i] = __floats2bfloat162_rn(f[i].x, f[i].y);
  } else if constexpr (std::is_same<T, __half>::value) {
    __half2* o = reinterpret_cast<__half2*>(v.v);
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) o[i] = __floats2half2_rn(f[i].x, f[i].y);
  } else {
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      v.v[2 * i] = f[i].x;
      v.v[2 * i + 1] = f[i].y;
    }
  }
}

// CTA-wide sums of Q quantities for N rows with the per-row epilogue folded in: after the
// exchange lane l owns the total of row (l % N) for each quantity, `post(q, total)` is applied
// there once, and the results are broadcast so that every thread returns with all N values
// in v[q][*]. `mine[q]` keeps the lane's own value (row l % N), which lets N lanes of warp 0
// write per-row statistics without any further exchange. Fixed summation order; callers
// alternate between two `red` buffers (one __syncthreads per call).
template <int Q, int N, class Post>
__device__ __forceinline__ void cta_sum_rows_post(float (&v)[Q][N], float (&mine)[Q], float* red, int lane, int warp,
                                                  int warps, Post post) {
  constexpr int kLanesPerRow = 32 / N;
#pragma unroll
  for (int q = 0; q < Q; ++q) {
    warp_sum_rows<N>(v[q], lane);
    if ((lane & (kLanesPerRow - 1)) == 0) red[(q * N + row_of_lane<N>(lane)) * 32 + warp] = v[q][0];
  }
  __syncthreads();
  const int row = lane & (N - 1), slot = lane / N;
#pragma unroll
  for (int q = 0; q < Q; ++q) {
    const float* src = red + (q * N + row) * 32;
    float t = slot < warps ? src[slot] : 0.f;
    if (warps > kLanesPerRow) {
      for (int w = slot + kLanesPerRow; w < warps; w += kLanesPerRow) t += src[w];
    }
#pragma unroll
    for (int width = 16; width >= N; width >>= 1) t += __shfl_xor_sync(0xffffffffu, t, width);
    t = post(q, t);
    mine[q] = t;
#pragma unroll
    for (int j = 0; j < N; ++j) v[q][j] = __shfl_sync(0xffffffffu, t, j);
  }
}

// 1/sqrt(x) from the 2-ulp hardware approximation plus one Newton step (about 1 ulp), without
// the slow-path branches of an IEEE sqrt followed by an IEEE divide.
__device__ __forceinline__ float rsqrt_newton(float x) {
  const float r = rsqrtf(x);
  return r * fmaf(-0.5f * x, r * r, 1.5f);
}

}  // namespace nd
