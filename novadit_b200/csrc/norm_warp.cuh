// AdaLN / AdaRMSNorm FORWARD with one warp per row (sm_100a).
//
// Why a second forward kernel. In the CTA-per-row-group kernels of norm_tma.cuh every warp of the CTA pays
// the per-row costs - two CTA-wide reductions, the statistics, loop and address arithmetic - for every row,
// although it only holds a fifth of the row: 630 warp instructions per row at H = 1152, of which ~200 touch
// data. Here a warp owns a whole row: the row sums are two 5-step shuffle butterflies, nothing is replicated,
// warps never wait for each other inside a sample, and the count drops to about a third. Measured on B200 at
// H = 1152 bf16: 5.75 TB/s against 5.46 at 131 072 rows, but 10 % SLOWER at 8192 and 32 768 rows, where the
// time goes to launch, first-byte latency and the tail rather than to instructions - so the launcher uses
// this kernel for large tensors only.
//
// Work split and data path are those of norm_tma.cuh: one chunk of rows per CTA, groups of up to 4 rows that
// stay inside one sample, one cp.async.bulk per group into a shared-memory ring, completion on an mbarrier.
// A CTA has 4 warps, warp w takes row w of the group. A stage is handed back through an "empty" mbarrier that
// every warp arrives on once its row sits in registers; thread 0 then sends the next group into the stage of the
// PREVIOUS group, so it practically never waits. The modulation vectors of the sample, (1 + scale) and shift, are kept in shared
// memory as fp32 and re-read per row (a lane's 36 columns would not fit in registers twice more).
// Lane l of a warp owns the 16-byte vectors l, l + 32, ... of its row: NV of them, the last pass partly idle.
// Numerics are those of the other kernels: two-pass variance over registers in fp32, rsqrt + one Newton
// step, one rounding on store. Every mbarrier wait is bounded (1 s).
#pragma once

#include <cuda_fp8.h>

#include "norm_tma.cuh"

namespace nd {

constexpr int kWarpRows = 4;     // rows per group = warps per CTA
constexpr int kWarpThreads = 32 * kWarpRows;

// bytes of dynamic shared memory: full barriers | modulation (4 float4 arrays of nvec) | stages
__host__ __device__ inline size_t norm_warp_smem(int hidden, int elem_bytes, int stages) {
  const size_t mod = static_cast<size_t>(hidden) * 2 * sizeof(float);
  return kBarrierBytes + mod + static_cast<size_t>(stages) * kWarpRows * hidden * elem_bytes;
}

#ifndef ND_WARP_MINB
#define ND_WARP_MINB 5
#endif
// Q8: the output is FP8 e4m3 (one byte per element) under a caller-given scale, and the largest |value| of the
// launch is folded into a device float with an atomic max - the delayed-scaling recipe: this step quantises with
// the scale derived from an earlier step's maximum and records its own for the next one, so the activation
// never exists in 16 bits and FC1's FP8 operand needs no separate amax / quantise pass.
template <typename T, int VEC, int NV, bool RMS, bool Q8 = false>
__global__ void __launch_bounds__(kWarpThreads, ND_WARP_MINB) norm_fwd_warp(const NormArgs a) {
  constexpr int NP = VEC / 2;   // float2 pairs per vector
  constexpr int NF4 = VEC / 4;  // float4 chunks per vector
  constexpr int RPI = kWarpRows;
  extern __shared__ __align__(128) unsigned char dsm[];
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm);
  __shared__ uint64_t empty[kMaxStages];
  __shared__ int s_abort;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = a.hidden;
  const int nvec = H / VEC;
  // modulation in shared memory: [scale | shift][float4 chunk k][vector v], so that consecutive lanes read
  // consecutive 16-byte words
  float4* mod = reinterpret_cast<float4*>(dsm + kBarrierBytes);
  unsigned char* buf = dsm + kBarrierBytes + static_cast<size_t>(H) * 2 * sizeof(float);
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const uint32_t stage_total = RPI * row_bytes;
  const float inv_h = 1.f / static_cast<float>(H);
  const float eps = a.eps;
  const int stages = a.stages;
  const bool tail_valid = (NV - 1) * 32 + lane < nvec;  // the last pass covers the ragged end of the row

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], RPI);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  griddep_launch_dependents();
  __syncthreads();
  griddep_wait();  // nothing above reads global memory; everything below may

  GroupCursor pc;
  bool pc_valid = false;
  if (tid == 0) {
    // stages - 1 groups go out now, the next one whenever a group has been read: a smaller first burst reaches
    // the CTAs sooner (all CTAs of the wave ask at once, and the last byte of the burst arrives with the first)
    pc_valid = pc.init(a);
    for (int s = 0; s < stages - 1 && pc_valid; ++s) {
      issue_group<T, RPI, false>(a, pc, s, full, buf, row_bytes);
      pc_valid = pc.next(a, RPI);
    }
  }

  [[maybe_unused]] float q_inv = 1.f, q_max = 0.f;
  if constexpr (Q8) q_inv = 1.f / __ldg(a.q_scale);

  int stage = 0;
  uint32_t parity = 0;          // phase of full[stage] to wait for
  int prev_stage = -1;          // stage of the previous group (refilled by thread 0)
  uint32_t prev_parity = 0;     // phase of empty[prev_stage] that its readers complete
  GroupCursor cc;
  bool more = cc.init(a);
  while (more) {
    const long long b = cc.b;
    // the sample's modulation -> shared memory as fp32 (1 + scale, shift); all warps have left the previous sample
    __syncthreads();
    for (int v = tid; v < nvec; v += kWarpThreads) {
      Vec<T, VEC> vs, vh;
      vs.load(static_cast<const T*>(a.scale) + b * H + v * VEC);
      vh.load(static_cast<const T*>(a.shift) + b * H + v * VEC);
      float2 sc[NP], sh[NP];
      unpack2<T, VEC>(vs, sc);
      unpack2<T, VEC>(vh, sh);
#pragma unroll
      for (int k = 0; k < NF4; ++k) {
        mod[(0 * NF4 + k) * nvec + v] = make_float4(1.f + sc[2 * k].x, 1.f + sc[2 * k].y, 1.f + sc[2 * k + 1].x, 1.f + sc[2 * k + 1].y);
        mod[(1 * NF4 + k) * nvec + v] = make_float4(sh[2 * k].x, sh[2 * k].y, sh[2 * k + 1].x, sh[2 * k + 1].y);
      }
    }
    __syncthreads();

    do {
      const long long r = cc.r;
      const int nrows = cc.group_rows(RPI);
      if (*static_cast<volatile int*>(&s_abort)) {
        drain_after_abort();
        return;
      }
      if (!mbar_wait_1s(&full[stage], parity, a.err, 1)) {
        s_abort = 1;
        drain_after_abort();
        return;
      }
      const bool mine = warp < nrows;  // this warp has a row in the group
      float2 X[NV][NP];
      if (mine) {
        const unsigned char* src = buf + static_cast<size_t>(stage) * stage_total + warp * row_bytes;
#pragma unroll
        for (int p = 0; p < NV; ++p) {
          const int v = p * 32 + lane;
          Vec<T, VEC> pk;
          if (p < NV - 1 || tail_valid) {
            *reinterpret_cast<uint4*>(pk.v) = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(v) * 16);
          } else {
            pk.zero();
          }
          unpack2<T, VEC>(pk, X[p]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);  // this warp's row has left the stage
      if (tid == 0 && pc_valid) {
        // the next group goes into the stage behind this one in the ring: never used in the first iteration,
        // afterwards the previous group's stage, whose readers arrived an iteration ago
        const int target = prev_stage >= 0 ? prev_stage : stages - 1;
        if (prev_stage >= 0 && !mbar_wait_1s(&empty[prev_stage], prev_parity, a.err, 3)) {
          s_abort = 1;
        } else {
          if (prev_stage >= 0) fence_proxy_async_smem();
          issue_group<T, RPI, false>(a, pc, target, full, buf, row_bytes);
          pc_valid = pc.next(a, RPI);
        }
      }
      __syncwarp();

      if (mine) {
        float mean = 0.f;
        if constexpr (!RMS) {
          float2 acc = X[0][0];
#pragma unroll
          for (int p = 0; p < NV; ++p) {
#pragma unroll
            for (int i = (p == 0 ? 1 : 0); i < NP; ++i) acc = __fadd2_rn(acc, X[p][i]);
          }
          float s = acc.x + acc.y;
#pragma unroll
          for (int w = 16; w >= 1; w >>= 1) s += __shfl_xor_sync(0xffffffffu, s, w);
          mean = s * inv_h;
          const float2 nm = make_float2(-mean, -mean);
#pragma unroll
          for (int p = 0; p < NV; ++p) {
            if (p < NV - 1 || tail_valid) {  // the idle lanes of the last pass keep zeros: they add nothing below
#pragma unroll
              for (int i = 0; i < NP; ++i) X[p][i] = __fadd2_rn(X[p][i], nm);  // deviations, in place
            }
          }
        }
        float2 acc2 = __fmul2_rn(X[0][0], X[0][0]);
#pragma unroll
        for (int p = 0; p < NV; ++p) {
#pragma unroll
          for (int i = (p == 0 ? 1 : 0); i < NP; ++i) acc2 = __ffma2_rn(X[p][i], X[p][i], acc2);
        }
        float q = acc2.x + acc2.y;
#pragma unroll
        for (int w = 16; w >= 1; w >>= 1) q += __shfl_xor_sync(0xffffffffu, q, w);
        const float rstd = rsqrt_newton(fmaf(q, inv_h, eps));
        if (lane == 0 && a.invstd != nullptr) {
          if constexpr (!RMS) a.mean[r + warp] = mean;
          a.invstd[r + warp] = rstd;
        }
        const float2 r2 = make_float2(rstd, rstd);
        T* yrow = static_cast<T*>(a.y) + (r + warp) * static_cast<long long>(H);
#pragma unroll
        for (int p = 0; p < NV; ++p) {
          const int v = p * 32 + lane;
          if (p < NV - 1 || tail_valid) {
            float2 out[NP];
#pragma unroll
            for (int k = 0; k < NF4; ++k) {
              const float4 s4 = mod[(0 * NF4 + k) * nvec + v], h4 = mod[(1 * NF4 + k) * nvec + v];
              out[2 * k] = __ffma2_rn(__fmul2_rn(X[p][2 * k], r2), make_float2(s4.x, s4.y), make_float2(h4.x, h4.y));
              out[2 * k + 1] = __ffma2_rn(__fmul2_rn(X[p][2 * k + 1], r2), make_float2(s4.z, s4.w), make_float2(h4.z, h4.w));
            }
            if constexpr (Q8) {
              unsigned short pk[NP];
#pragma unroll
              for (int i = 0; i < NP; ++i) {
                q_max = fmaxf(q_max, fmaxf(fabsf(out[i].x), fabsf(out[i].y)));
                pk[i] = __nv_cvt_float2_to_fp8x2(make_float2(out[i].x * q_inv, out[i].y * q_inv), __NV_SATFINITE, __NV_E4M3);
              }
              unsigned char* qrow = static_cast<unsigned char*>(a.y) + (r + warp) * static_cast<long long>(H);
              if constexpr (VEC == 8) {
                *reinterpret_cast<uint2*>(qrow + static_cast<long long>(v) * 8) =
                    make_uint2(pk[0] | (static_cast<uint32_t>(pk[1]) << 16), pk[2] | (static_cast<uint32_t>(pk[3]) << 16));
              } else {
                *reinterpret_cast<uint32_t*>(qrow + static_cast<long long>(v) * 4) = pk[0] | (static_cast<uint32_t>(pk[1]) << 16);
              }
            } else {
              Vec<T, VEC> o;
              pack2<T, VEC>(out, o);
              o.store(yrow + static_cast<long long>(v) * VEC);
            }
          }
        }
      }

      prev_stage = stage;
      prev_parity = parity;
      if (++stage == stages) {
        stage = 0;
        parity ^= 1u;
      }
      more = cc.next(a, RPI);
    } while (more && cc.b == b);
  }
  if constexpr (Q8) {
    if (a.q_amax != nullptr) {
#pragma unroll
      for (int w = 16; w >= 1; w >>= 1) q_max = fmaxf(q_max, __shfl_xor_sync(0xffffffffu, q_max, w));
      // non-negative floats order like their bit patterns: an integer max is a float max, and it is exact
      if (lane == 0) atomicMax(reinterpret_cast<int*>(a.q_amax), __float_as_int(q_max));
    }
  }
}

}  // namespace nd
