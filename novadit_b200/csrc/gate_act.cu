// Gated activation y = up * act(gate), rows [up(I) | gate(I)], forward and backward (sm_100a).
//
// Pure streaming work. One CTA per group of RG rows (RG = 1 for rows of 8 KB and more); thread t handles
// column vectors t, t + NT, ... of the group's rows with the loads of all passes issued up front, so
// 2 (forward) or 3 (backward) x RG x passes independent 128-bit loads are in flight per thread and no index
// division is needed. Math is fp32, rounded once on store.
#include <atomic>

#include "common.cuh"

namespace nd {

struct GateArgs {
  const void* x;   // [rows, 2I]
  const void* dy;  // [rows, I] (backward)
  void* out;       // y [rows, I] or dz [rows, 2I]
  long long rows;
  int inter;
  int gate_first;  // 0: rows are [up | gate] (the gate-act operator); 1: rows are [gate | up] (FC1's z = x W^T + b)
};

// PASSES > 0: the row needs exactly that many passes of the CTA's threads and all of them are unrolled, so
// the loads of every pass are issued before the first result is stored; PASSES == 0: any width, plain loop.
template <typename T, int VEC, int RG, int ACT, bool BWD, int PASSES, int MAXT = 256>
__global__ void __launch_bounds__(MAXT) gate_act_kernel(const GateArgs a) {
  const int I = a.inter;
  const int nvec = I / VEC;
  const T* __restrict__ x = static_cast<const T*>(a.x);
  const T* __restrict__ dy = static_cast<const T*>(a.dy);
  T* __restrict__ out = static_cast<T*>(a.out);
  const long long groups = (a.rows + RG - 1) / RG;
  const long long in_stride = 2LL * I;
  const long long out_stride = BWD ? 2LL * I : I;
  const int up_off = a.gate_first ? I : 0, gate_off = a.gate_first ? 0 : I;  // halves of an input / dz row
  constexpr int NP = PASSES > 0 ? PASSES : 1;

  for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
    const long long r0 = g * RG;
    for (int iv0 = threadIdx.x; iv0 < (PASSES > 0 ? static_cast<int>(blockDim.x) : nvec); iv0 += blockDim.x) {
      Vec<T, VEC> up[NP][RG], gate[NP][RG], gy[NP][RG];
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        const int iv = iv0 + p * static_cast<int>(blockDim.x);
        const int col = iv * VEC;
#pragma unroll
        for (int j = 0; j < RG; ++j) {
          up[p][j].zero();
          gate[p][j].zero();
          if constexpr (BWD) gy[p][j].zero();
          if (iv < nvec && r0 + j < a.rows) {
            const T* row = x + (r0 + j) * in_stride;
            up[p][j].load_stream(row + up_off + col);
            gate[p][j].load_stream(row + gate_off + col);
            if constexpr (BWD) gy[p][j].load_stream(dy + (r0 + j) * I + col);
          }
        }
      }
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        const int iv = iv0 + p * static_cast<int>(blockDim.x);
        const int col = iv * VEC;
#pragma unroll
        for (int j = 0; j < RG; ++j) {
          if (iv < nvec && r0 + j < a.rows) {
            float fu[VEC], fg[VEC];
            up[p][j].unpack(fu);
            gate[p][j].unpack(fg);
            if constexpr (!BWD) {
              float fy[VEC];
#pragma unroll
              for (int k = 0; k < VEC; ++k) fy[k] = fu[k] * act_fwd<ACT>(fg[k]);
              Vec<T, VEC> o;
              o.pack(fy);
              o.store(out + (r0 + j) * out_stride + col);
            } else {
              float fd[VEC], du[VEC], dg[VEC];
              gy[p][j].unpack(fd);
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
              o0.store(orow + up_off + col);
              o1.store(orow + gate_off + col);
            }
          }
        }
      }
    }
  }
}

template <typename T, int VEC, int RG, int PASSES>
static const void* pick_gate_kernel_p(int act, bool bwd) {
  if (act == ND_ACT_SILU)
    return bwd ? (const void*)gate_act_kernel<T, VEC, RG, ND_ACT_SILU, true, PASSES>
               : (const void*)gate_act_kernel<T, VEC, RG, ND_ACT_SILU, false, PASSES>;
  return bwd ? (const void*)gate_act_kernel<T, VEC, RG, ND_ACT_GELU, true, PASSES>
             : (const void*)gate_act_kernel<T, VEC, RG, ND_ACT_GELU, false, PASSES>;
}

// GELU backward of one row per CTA in TWO unrolled passes of up to 320 threads (see launch_gate_rg)
template <typename T, int VEC>
static const void* pick_gate_kernel_wide() {
  return (const void*)gate_act_kernel<T, VEC, 1, ND_ACT_GELU, true, 2, 320>;
}

// unrolled passes only while the loads in flight stay within the register budget (RG * passes <= 4)
template <typename T, int VEC, int RG>
static const void* pick_gate_kernel(int act, bool bwd, int passes) {
  // GELU backward carries the most registers per element in flight: with nine loads per thread (one row, three
  // unrolled passes) it loses occupancy (240 us at the 32 768 x 4608 shape against 225 us for the plain loop)
  if (bwd && act == ND_ACT_GELU && passes > 2) return pick_gate_kernel_p<T, VEC, RG, 0>(act, bwd);
  if (passes == 1) return pick_gate_kernel_p<T, VEC, RG, 1>(act, bwd);
  if constexpr (RG <= 2) {
    if (passes == 2) return pick_gate_kernel_p<T, VEC, RG, 2>(act, bwd);
  }
  if constexpr (RG == 1) {
    if (passes == 3) return pick_gate_kernel_p<T, VEC, RG, 3>(act, bwd);
    if (passes == 4) return pick_gate_kernel_p<T, VEC, RG, 4>(act, bwd);
  }
  return pick_gate_kernel_p<T, VEC, RG, 0>(act, bwd);
}

static std::atomic<int> g_gate_rows{0};     // rows per group: 0 = built-in choice
static std::atomic<int> g_gate_persist{0};  // 1 = one wave of CTAs striding over the groups

template <typename T, int RG>
static int launch_gate_rg(GateArgs a, int act, bool bwd, cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(T);
  bool vec_ok = (a.inter % VMAX) == 0 && aligned16(a.x) && aligned16(a.out) && aligned16(a.dy);
  const int nvec = vec_ok ? a.inter / VMAX : a.inter;
  // threads: spread the row's vectors evenly over the fewest passes of <= 256 threads
  const int passes = (nvec + 255) / 256;
  int nt = ((nvec + passes - 1) / passes + 31) / 32 * 32;
  if (nt < 32) nt = 32;
  const void* fn = vec_ok ? pick_gate_kernel<T, VMAX, RG>(act, bwd, passes) : pick_gate_kernel<T, 1, RG>(act, bwd, passes);
  if constexpr (RG == 1) {
    // GELU backward of a row of three passes (513..640 vectors: I = 4608 in 16-bit types is 576): three unrolled
    // passes (nine loads per thread) cost occupancy and the plain loop waits for its loads three times in a row;
    // two unrolled passes of 288 threads (six loads per thread) measured 3 % faster than either (219 against 226 us
    // at 32 768 x 4608, fwd + bwd 349 us = 6.9 TB/s)
    if (vec_ok && bwd && act == ND_ACT_GELU && passes == 3 && nvec <= 640) {
      nt = ((nvec + 1) / 2 + 31) / 32 * 32;
      fn = pick_gate_kernel_wide<T, VMAX>();
    }
  }
  const long long groups = (a.rows + RG - 1) / RG;
  // One CTA per group of rows: tens of thousands of short CTAs that the hardware scheduler hands to whichever
  // SM frees up first. A single resident wave striding over the groups left every CTA with 11 or 12 groups at
  // the 32 768-row shape - an 8 % tail - and measured 12 % slower.
  long long grid = groups;
  if (g_gate_persist.load(std::memory_order_relaxed) != 0) {
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, nt, 0) != cudaSuccess || occ < 1) {
      (void)cudaGetLastError();
      occ = 1;
    }
    grid = static_cast<long long>(sm_count()) * occ;
    if (grid > groups) grid = groups;
  }
  if (grid > 0x7FFFFFFFLL) grid = 0x7FFFFFFFLL;  // the kernel strides, so a capped grid still covers every group
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

template <typename T>
static int launch_gate(GateArgs a, int act, bool bwd, cudaStream_t st) {
  // rows per CTA: one where a row is a CTA's worth of work (8 KB and up), more for narrow rows
  int rg = g_gate_rows.load(std::memory_order_relaxed);
  if (rg <= 0) {
    const long long row_bytes = static_cast<long long>(a.inter) * sizeof(T);
    rg = row_bytes >= 8192 ? 1 : row_bytes >= 4096 ? 2 : 4;
  }
  switch (rg) {
    case 1: return launch_gate_rg<T, 1>(a, act, bwd, st);
    case 2: return launch_gate_rg<T, 2>(a, act, bwd, st);
    default: return launch_gate_rg<T, 4>(a, act, bwd, st);
  }
}

static int gate_entry(int dtype, int act, bool bwd, const void* dy, const void* x, void* out,
                      int64_t rows, int64_t inter, void* stream, int gate_first = 0) {
  if (rows < 0 || inter <= 0) return ND_ERR_BAD_ARG;
  if (act != ND_ACT_SILU && act != ND_ACT_GELU) return ND_ERR_UNSUPPORTED;
  if (inter > INT32_MAX / 2) return ND_ERR_UNSUPPORTED;
  if (rows == 0) return ND_OK;
  if (!x || !out || (bwd && !dy)) return ND_ERR_BAD_ARG;
  GateArgs a{x, dy, out, rows, static_cast<int>(inter), gate_first != 0 ? 1 : 0};
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

// Tuning hook: rows per CTA group (1, 2 or 4; 0 = built-in choice) and whether a single resident wave of CTAs
// strides over the groups (1) or every group gets its own CTA (0, default). Process-wide.
void nd_tune_gate_act(int rows_per_group, int persistent) {
  nd::g_gate_rows.store(rows_per_group);
  nd::g_gate_persist.store(persistent != 0);
}

int nd_gate_act_fwd(int dtype, int act, const void* x, void* y, int64_t rows, int64_t inter,
                    void* stream) {
  return nd::gate_entry(dtype, act, false, nullptr, x, y, rows, inter, stream);
}

int nd_gate_act_bwd(int dtype, int act, const void* dy, const void* x, void* dz, int64_t rows,
                    int64_t inter, void* stream) {
  return nd::gate_entry(dtype, act, true, dy, x, dz, rows, inter, stream);
}

// The same backward for rows laid out [gate(I) | up(I)], which is FC1's pre-activation z = x W^T + b with the
// nn.Linear weight as stored: dz = [dy * up * act'(gate) | dy * act(gate)].
int nd_gate_act_bwd_gate_first(int dtype, int act, const void* dy, const void* z, void* dz, int64_t rows,
                               int64_t inter, void* stream) {
  return nd::gate_entry(dtype, act, true, dy, z, dz, rows, inter, stream, 1);
}

}  // extern "C"
