// Shared device/host helpers for the sm_100a operator kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "../../include/novadit_b200.h"
#include "../../include/novadit_b200_tuning.h"

namespace nd {

// ---------------------------------------------------------------- host side
void set_last_cuda_error(cudaError_t e);

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}

int sm_count();  // multiprocessors of the current device (cached per device)
int* device_error_ptr();  // device address of the error word kernels set when a bounded wait expires

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// -------------------------------------------------------------- conversions
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// A vector of VEC elements moved with one load/store of VEC*sizeof(T) bytes.
template <int BYTES> struct RawOf;
template <> struct RawOf<16> { using type = uint4; };
template <> struct RawOf<8> { using type = uint2; };
template <> struct RawOf<4> { using type = uint32_t; };
template <> struct RawOf<2> { using type = uint16_t; };
template <> struct RawOf<1> { using type = uint8_t; };

template <typename T, int VEC> struct alignas(sizeof(T) * VEC) Vec {
  using Raw = typename RawOf<sizeof(T) * VEC>::type;
  T v[VEC];

  __device__ __forceinline__ void load(const T* p) {
    *reinterpret_cast<Raw*>(v) = __ldg(reinterpret_cast<const Raw*>(p));
  }
  __device__ __forceinline__ void load_stream(const T* p) {  // read-once data: do not keep in L1
    *reinterpret_cast<Raw*>(v) = __ldcs(reinterpret_cast<const Raw*>(p));
  }
  __device__ __forceinline__ void store(T* p) const {
    *reinterpret_cast<Raw*>(p) = *reinterpret_cast<const Raw*>(v);
  }
  // Make the register contents opaque to the optimiser. Used between two passes over the same
  // packed data so that the second pass converts from the packed registers again instead of
  // keeping every fp32 copy of the first pass alive (which multiplies the register footprint).
  __device__ __forceinline__ void opaque() {
    if constexpr (sizeof(T) * VEC >= 4) {
      uint32_t* w = reinterpret_cast<uint32_t*>(v);
#pragma unroll
      for (int i = 0; i < static_cast<int>(sizeof(T) * VEC / 4); ++i) asm volatile("" : "+r"(w[i]));
    } else {
      uint16_t* w = reinterpret_cast<uint16_t*>(v);
      asm volatile("" : "+h"(w[0]));
    }
  }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = from_f32<T>(0.f);
  }
  __device__ __forceinline__ void unpack(float (&f)[VEC]) const {
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = to_f32(v[i]);
  }
  __device__ __forceinline__ void pack(const float (&f)[VEC]) {
    if constexpr (sizeof(T) == 2 && VEC % 2 == 0) {
#pragma unroll
      for (int i = 0; i < VEC; i += 2) {
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          *reinterpret_cast<__nv_bfloat162*>(&v[i]) = __floats2bfloat162_rn(f[i], f[i + 1]);
        } else {
          *reinterpret_cast<__half2*>(&v[i]) = __floats2half2_rn(f[i], f[i + 1]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = from_f32<T>(f[i]);
    }
  }
};

// ------------------------------------------------------------ row reductions
// Sum N per-lane values (one per row) over the 32 lanes of a warp with a
// transposed butterfly: the first log2(N) steps exchange half of the values
// each, so N values cost N-1 + (5 - log2 N) shuffles instead of 5N. On return
// v[0] of lane l holds the warp total of row row_of_lane<N>(l).
template <int N> __device__ __forceinline__ int row_of_lane(int lane) {
  int r = 0;
  int width = 16;
#pragma unroll
  for (int n = N; n > 1; n >>= 1, width >>= 1) r += (lane & width) ? (n >> 1) : 0;
  return r;
}

template <int N> __device__ __forceinline__ void warp_sum_rows(float (&v)[N], int lane) {
  static_assert(N == 1 || N == 2 || N == 4 || N == 8 || N == 16, "N must be a power of two <= 16");
  int width = 16;
#pragma unroll
  for (int n = N; n > 1; n >>= 1) {
    const int half = n >> 1;
    const bool upper = (lane & width) != 0;
#pragma unroll
    for (int j = 0; j < half; ++j) {
      const float send = upper ? v[j] : v[j + half];
      const float keep = upper ? v[j + half] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, width);
    }
    width >>= 1;
  }
#pragma unroll
  for (; width >= 1; width >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], width);
}

// CTA-wide sums of Q quantities for N rows. `red` is shared memory of
// Q * N * 32 floats whose slots [q][row][w >= warps] are zero. Every thread
// returns with the totals of all rows, summed over warps in a fixed order.
// Two calls that reuse the same `red` must be separated by a call on another
// buffer (callers alternate between two buffers), which is what makes one
// __syncthreads per call enough.
template <int Q, int N>
__device__ __forceinline__ void cta_sum_rows(float (&v)[Q][N], float* red, int lane, int warp,
                                             int warps) {
#pragma unroll
  for (int q = 0; q < Q; ++q) {
    warp_sum_rows<N>(v[q], lane);
    constexpr int kLanesPerRow = 32 / N;  // lanes holding the same row after the butterfly
    if ((lane & (kLanesPerRow - 1)) == 0) red[(q * N + row_of_lane<N>(lane)) * 32 + warp] = v[q][0];
  }
  __syncthreads();
  const int w4 = (warps + 3) >> 2;
#pragma unroll
  for (int q = 0; q < Q; ++q) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const float4* src = reinterpret_cast<const float4*>(red + (q * N + j) * 32);
      float s = 0.f;
      for (int w = 0; w < w4; ++w) {
        const float4 t = src[w];
        s += t.x;
        s += t.y;
        s += t.z;
        s += t.w;
      }
      v[q][j] = s;
    }
  }
}

// x * sigmoid(t): the common form of SiLU (t = x) and tanh-GELU (t = 2u). sigmoid = 1 / (1 + 2^(-t log2 e))
// from the two special-function instructions directly (ex2.approx: 2 ulp, rcp.approx: 1 ulp; flush-to-zero,
// +inf -> 0), so that the value before the output rounding stays within ~1e-6 relative of the exact one
// (tanh.approx, at 5e-4 absolute, would flip output roundings against the fp32 reference). Four instructions
// per sigmoid; the library exp2f / division would add range fix-ups that the formula does not need.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 1 / (1 + 2^e)
__device__ __forceinline__ float sigmoid_from_exp2arg(float e) { return rcp_approx(1.f + ex2_approx(e)); }
__device__ __forceinline__ float sigmoid_f32(float t) { return sigmoid_from_exp2arg(-1.4426950408889634f * t); }

constexpr float kGeluC0 = 0.7978845608028654f;  // sqrt(2/pi)
constexpr float kGeluC1 = 0.044715f;
// tanh-GELU: 0.5 g (1 + tanh u) == g * sigmoid(2u), u = c0 (g + c1 g^3); exponent argument -2 log2(e) u
constexpr float kGeluE0 = -2.f * 1.4426950408889634f * kGeluC0;
constexpr float kGeluE1 = kGeluE0 * kGeluC1;

template <int ACT> __device__ __forceinline__ float act_fwd(float g) {
  if constexpr (ACT == ND_ACT_NONE) {
    return g;
  } else if constexpr (ACT == ND_ACT_SILU) {
    return g * sigmoid_f32(g);
  } else {
    return g * sigmoid_from_exp2arg(g * fmaf(kGeluE1, g * g, kGeluE0));
  }
}

// One special-function instruction per activation instead of two: x * sigmoid(t) = h (1 + tanh(t / 2)) with h = x / 2
// and the hardware tanh (absolute error ~5e-4 of the tanh, i.e. of the gate factor). Too coarse for the 16-bit
// operators' parity bars; used where the operands are FP8 (whose quantisation noise is two orders of magnitude
// larger) and the epilogue is bound by the special-function unit.
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int ACT> __device__ __forceinline__ float act_fwd_fast(float g) {
  if constexpr (ACT == ND_ACT_NONE) {
    return g;
  } else if constexpr (ACT == ND_ACT_SILU) {
    const float h = 0.5f * g;
    return fmaf(h, tanh_approx(h), h);
  } else {
    const float h = 0.5f * g;
    return fmaf(h, tanh_approx(g * fmaf(kGeluC0 * kGeluC1, g * g, kGeluC0)), h);
  }
}

// returns act(g) and writes act'(g)
template <int ACT> __device__ __forceinline__ float act_fwd_grad(float g, float& grad) {
  if constexpr (ACT == ND_ACT_SILU) {
    const float s = sigmoid_f32(g);
    grad = s * (1.f + g * (1.f - s));
    return g * s;
  } else {
    const float g2 = g * g;
    const float s = sigmoid_from_exp2arg(g * fmaf(kGeluE1, g2, kGeluE0));  // = 0.5 (1 + tanh u)
    // d/dg [g s] = s + g * s' ,  s' = 2 s (1 - s) * du/dg
    const float du = kGeluC0 * (1.f + 3.f * kGeluC1 * g2);
    grad = s + g * 2.f * s * (1.f - s) * du;
    return g * s;
  }
}

}  // namespace nd
