// Gated activation y = up * act(gate), rows [up(I) | gate(I)], forward and backward (sm_100a).
//
// Pure streaming work. A CTA walks groups of RG rows; within a group thread t
// handles column vector t, t + NT, ... of all RG rows, so 2*RG (forward) or
// 3*RG (backward) independent 128-bit loads are in flight per thread and no
// index division is needed. Math is fp32, rounded once on store.
#include "common.cuh"

namespace nd {

struct GateArgs {
  const void* x;   // [rows, 2I]
  const void* dy;  // [rows, I] (backward)
  void* out;       // y [rows, I] or dz [rows, 2I]
  long long rows;
  int inter;
};

template <typename T, int VEC, int RG, int ACT, bool BWD>
__global__ void __launch_bounds__(256) gate_act_kernel(const GateArgs a) {
  const int I = a.inter;
  const int nvec = I / VEC;
  const T* __restrict__ x = static_cast<const T*>(a.x);
  const T* __restrict__ dy = static_cast<const T*>(a.dy);
  T* __restrict__ out = static_cast<T*>(a.out);
  const long long groups = (a.rows + RG - 1) / RG;
  const long long in_stride = 2LL * I;
  const long long out_stride = BWD ? 2LL * I : I;

  for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
    const long long r0 = g * RG;
    for (int iv = threadIdx.x; iv < nvec; iv += blockDim.x) {
      const int col = iv * VEC;
      Vec<T, VEC> up[RG], gate[RG], gy[RG];
#pragma unroll
      for (int j = 0; j < RG; ++j) {
        up[j].zero();
        gate[j].zero();
        if constexpr (BWD) gy[j].zero();
        if (r0 + j < a.rows) {
          const T* row = x + (r0 + j) * in_stride;
          up[j].load_stream(row + col);
          gate[j].load_stream(row + I + col);
          if constexpr (BWD) gy[j].load_stream(dy + (r0 + j) * I + col);
        }
      }
#pragma unroll
      for (int j = 0; j < RG; ++j) {
        if (r0 + j < a.rows) {
          float fu[VEC], fg[VEC];
          up[j].unpack(fu);
          gate[j].unpack(fg);
          if constexpr (!BWD) {
            float fy[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k) fy[k] = fu[k] * act_fwd<ACT>(fg[k]);
            Vec<T, VEC> o;
            o.pack(fy);
            o.store(out + (r0 + j) * out_stride + col);
          } else {
            float fd[VEC], du[VEC], dg[VEC];
            gy[j].unpack(fd);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
              float grad;
              const float av = act_fwd_grad<ACT>(fg[k], grad);
              du[k] = fd[k] * av;
              dg[k] = fd[k] * fu[k] * grad;
            }
            Vec<T, VEC> o0, o1;
            o0.pack(du);
            o1.pack(dg);
            T* orow = out + (r0 + j) * out_stride;
            o0.store(orow + col);
            o1.store(orow + I + col);
          }
        }
      }
    }
  }
}

template <typename T, int VEC, int RG>
static const void* pick_gate_kernel(int act, bool bwd) {
  if (act == ND_ACT_SILU)
    return bwd ? (const void*)gate_act_kernel<T, VEC, RG, ND_ACT_SILU, true>
               : (const void*)gate_act_kernel<T, VEC, RG, ND_ACT_SILU, false>;
  return bwd ? (const void*)gate_act_kernel<T, VEC, RG, ND_ACT_GELU, true>
             : (const void*)gate_act_kernel<T, VEC, RG, ND_ACT_GELU, false>;
}

template <typename T>
static int launch_gate(GateArgs a, int act, bool bwd, cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(T);
  bool vec_ok = (a.inter % VMAX) == 0 && aligned16(a.x) && aligned16(a.out) && aligned16(a.dy);
  const void* fn;
  int nvec;
  constexpr int RG = 4;
  if (vec_ok) {
    fn = pick_gate_kernel<T, VMAX, RG>(act, bwd);
    nvec = a.inter / VMAX;
  } else {
    fn = pick_gate_kernel<T, 1, RG>(act, bwd);
    nvec = a.inter;
  }
  // threads: spread the row's vectors evenly over the fewest passes of <= 256 threads
  const int passes = (nvec + 255) / 256;
  int nt = ((nvec + passes - 1) / passes + 31) / 32 * 32;
  if (nt < 32) nt = 32;
  const long long groups = (a.rows + RG - 1) / RG;
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, nt, 0) != cudaSuccess || occ < 1) {
    (void)cudaGetLastError();
    occ = 1;
  }
  long long grid = static_cast<long long>(sm_count()) * occ;
  if (grid > groups) grid = groups;
  if (grid < 1) return ND_OK;
  void* params[] = {&a};
  cudaError_t e = cudaLaunchKernel(fn, dim3(static_cast<unsigned>(grid)), dim3(nt), params, 0, st);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}

static int gate_entry(int dtype, int act, bool bwd, const void* dy, const void* x, void* out,
                      int64_t rows, int64_t inter, void* stream) {
  if (rows < 0 || inter <= 0) return ND_ERR_BAD_ARG;
  if (act != ND_ACT_SILU && act != ND_ACT_GELU) return ND_ERR_UNSUPPORTED;
  if (inter > INT32_MAX / 2) return ND_ERR_UNSUPPORTED;
  if (rows == 0) return ND_OK;
  if (!x || !out || (bwd && !dy)) return ND_ERR_BAD_ARG;
  GateArgs a{x, dy, out, rows, static_cast<int>(inter)};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case ND_F16: return launch_gate<__half>(a, act, bwd, st);
    case ND_BF16: return launch_gate<__nv_bfloat16>(a, act, bwd, st);
    case ND_F32: return launch_gate<float>(a, act, bwd, st);
    default: return ND_ERR_UNSUPPORTED;
  }
}

}  // namespace nd

extern "C" {

int nd_gate_act_fwd(int dtype, int act, const void* x, void* y, int64_t rows, int64_t inter,
                    void* stream) {
  return nd::gate_entry(dtype, act, false, nullptr, x, y, rows, inter, stream);
}

int nd_gate_act_bwd(int dtype, int act, const void* dy, const void* x, void* dz, int64_t rows,
                    int64_t inter, void* stream) {
  return nd::gate_entry(dtype, act, true, dy, x, dz, rows, inter, stream);
}

}  // extern "C"
