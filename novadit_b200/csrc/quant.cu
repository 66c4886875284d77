// Per-tensor FP8 e4m3 quantisation helpers for the FP8 FC1 path (sm_100a):
// a deterministic two-stage abs-max and a saturating scale-and-convert.
#include <cuda_fp8.h>

#include "common.cuh"

namespace nd {

constexpr int kAmaxCtas = 1024;  // stage-1 partial maxima (max is order-independent, so any grid works)
constexpr float kE4m3Max = 448.f;

template <typename T, int VEC>
__global__ void __launch_bounds__(256) amax_stage1_kernel(const T* __restrict__ x, long long n,
                                                          float* __restrict__ part) {
  __shared__ float smax[8];
  float m = 0.f;
  const long long nvec = n / VEC;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += 256LL * gridDim.x) {
    Vec<T, VEC> v;
    v.load_stream(x + i * VEC);
    float f[VEC];
    v.unpack(f);
#pragma unroll
    for (int k = 0; k < VEC; ++k) m = fmaxf(m, fabsf(f[k]));
  }
  // ragged tail (fewer than VEC elements) handled by one thread
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nvec * VEC; i < n; ++i) m = fmaxf(m, fabsf(to_f32(x[i])));
#pragma unroll
  for (int w = 16; w >= 1; w >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, w));
  if ((threadIdx.x & 31) == 0) smax[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = smax[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) r = fmaxf(r, smax[w]);
    part[blockIdx.x] = r;
  }
}

__global__ void __launch_bounds__(256) amax_stage2_kernel(const float* __restrict__ part, int count,
                                                          float* __restrict__ amax) {
  __shared__ float smax[8];
  float m = 0.f;
  for (int i = threadIdx.x; i < count; i += 256) m = fmaxf(m, part[i]);
#pragma unroll
  for (int w = 16; w >= 1; w >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, w));
  if ((threadIdx.x & 31) == 0) smax[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = smax[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) r = fmaxf(r, smax[w]);
    *amax = r;
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256) quant_e4m3_kernel(const T* __restrict__ x, long long n,
                                                         const float* __restrict__ amax,
                                                         __nv_fp8_storage_t* __restrict__ q,
                                                         float* __restrict__ scale_out) {
  const float am = *amax;
  const float scale = am > 0.f ? am / kE4m3Max : 1.f;  // de-quantisation scale
  const float inv = 1.f / scale;
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out != nullptr) *scale_out = scale;
  const long long nvec = n / VEC;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += 256LL * gridDim.x) {
    Vec<T, VEC> v;
    v.load_stream(x + i * VEC);
    float f[VEC];
    v.unpack(f);
    Vec<__nv_fp8_storage_t, VEC> o;
#pragma unroll
    for (int k = 0; k < VEC; ++k) o.v[k] = __nv_cvt_float_to_fp8(f[k] * inv, __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<typename RawOf<VEC>::type*>(q + i * VEC) =
        *reinterpret_cast<const typename RawOf<VEC>::type*>(o.v);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nvec * VEC; i < n; ++i)
      q[i] = __nv_cvt_float_to_fp8(to_f32(x[i]) * inv, __NV_SATFINITE, __NV_E4M3);
}

template <typename T>
static int launch_amax(const void* x, long long n, float* amax, float* part, cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(T);
  long long ctas = (n / VMAX + 255) / 256;
  if (ctas > kAmaxCtas) ctas = kAmaxCtas;
  if (ctas < 1) ctas = 1;
  if (aligned16(x))
    amax_stage1_kernel<T, VMAX><<<static_cast<unsigned>(ctas), 256, 0, st>>>(static_cast<const T*>(x), n, part);
  else
    amax_stage1_kernel<T, 1><<<static_cast<unsigned>(ctas), 256, 0, st>>>(static_cast<const T*>(x), n, part);
  amax_stage2_kernel<<<1, 256, 0, st>>>(part, static_cast<int>(ctas), amax);
  return check_launch();
}

template <typename T>
static int launch_quant(const void* x, long long n, const float* amax, void* q, float* scale_out,
                        cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(T);
  long long ctas = (n / VMAX + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  auto* qq = static_cast<__nv_fp8_storage_t*>(q);
  if (aligned16(x) && (reinterpret_cast<uintptr_t>(q) % VMAX) == 0)
    quant_e4m3_kernel<T, VMAX><<<static_cast<unsigned>(ctas), 256, 0, st>>>(static_cast<const T*>(x), n, amax, qq, scale_out);
  else
    quant_e4m3_kernel<T, 1><<<static_cast<unsigned>(ctas), 256, 0, st>>>(static_cast<const T*>(x), n, amax, qq, scale_out);
  return check_launch();
}

}  // namespace nd

extern "C" {

size_t nd_amax_ws_bytes(void) { return nd::kAmaxCtas * sizeof(float); }

int nd_amax(int dtype, const void* x, int64_t n, float* amax, void* ws, size_t ws_bytes,
            void* stream) {
  if (n < 0 || !amax || (n > 0 && !x)) return ND_ERR_BAD_ARG;
  if (!ws || ws_bytes < nd_amax_ws_bytes() || (reinterpret_cast<uintptr_t>(ws) & 255u)) return ND_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* part = static_cast<float*>(ws);
  switch (dtype) {
    case ND_F16: return nd::launch_amax<__half>(x, n, amax, part, st);
    case ND_BF16: return nd::launch_amax<__nv_bfloat16>(x, n, amax, part, st);
    case ND_F32: return nd::launch_amax<float>(x, n, amax, part, st);
    default: return ND_ERR_UNSUPPORTED;
  }
}

int nd_quant_e4m3(int dtype, const void* x, int64_t n, const float* amax, void* q,
                  float* scale_out, void* stream) {
  if (n < 0 || !amax || (n > 0 && (!x || !q))) return ND_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case ND_F16: return nd::launch_quant<__half>(x, n, amax, q, scale_out, st);
    case ND_BF16: return nd::launch_quant<__nv_bfloat16>(x, n, amax, q, scale_out, st);
    case ND_F32: return nd::launch_quant<float>(x, n, amax, q, scale_out, st);
    default: return ND_ERR_UNSUPPORTED;
  }
}

}  // extern "C"
