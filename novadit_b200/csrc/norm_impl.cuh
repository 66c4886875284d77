// AdaLN / AdaRMSNorm forward and backward kernels (sm_100a), shared by the
// per-dtype translation units norm_{f16,bf16,f32}.cu.
//
// Mapping. One CTA owns whole rows: thread i owns column vector i of 16 bytes
// (8 bf16/fp16 or 4 fp32; a scalar when the row is not 16-byte vectorisable)
// for RPI rows at a time, so RPI independent 128-bit loads per tensor are in
// flight per thread before the first is consumed. Row sums are reduced with a
// transposed warp butterfly plus one shared-memory exchange per RPI rows; the
// column sums of the backward pass (dscale / dshift) stay in the registers of
// the thread that owns the column, which is why no shared-memory or atomic
// reduction over rows is needed.
//
// Work items. The shard's rows are cut per sample into tiles of `tile_rows`
// rows; item = (sample, tile). All rows of an item share one sample, so the
// modulation vector is fetched once per item and kept in registers. The
// backward pass writes one fp32 partial [2, H] per item and the CTA that
// finishes a sample's last item sums the partials over tiles in index order
// (stage 2): deterministic, no floating-point atomics. The only atomic is the
// integer arrival counter per sample.
#pragma once

#include "common.cuh"

namespace nd {

enum NormMode { kFwd = 0, kBwdDx = 1, kBwdDparam = 2, kBwdFused = 3 };

struct NormArgs {
  const void* x;
  const void* scale;
  const void* shift;
  void* y;
  float* mean;    // LayerNorm mean per row (null for RMS, null for inference)
  float* invstd;  // 1/std (LayerNorm) or 1/rms (RMS) per row (null for inference)
  const void* dy;
  void* dx;
  float* dscale;
  float* dshift;
  float* ws_part;         // [n_items][2][hidden] fp32 partials (when tiles_per_sample > 1)
  unsigned int* ws_cnt;   // [n_samples] arrival counters, zero on entry and on exit
  long long rows, row_start;
  int seq_len, hidden;
  float eps;
  int tile_rows, tiles_per_sample;
  long long b_first, n_samples, n_items;
  int mode;
  bool rms;
};

// rows [l0, l1) (local to the shard) and sample b of a work item
__device__ __forceinline__ void item_rows(const NormArgs& a, long long item, long long& b,
                                          long long& bi, long long& l0, long long& l1) {
  bi = item / a.tiles_per_sample;
  const long long t = item - bi * a.tiles_per_sample;
  b = a.b_first + bi;
  const long long g0 = b * a.seq_len + t * a.tile_rows;
  long long g1 = g0 + a.tile_rows;
  const long long gend = (b + 1) * a.seq_len;
  if (g1 > gend) g1 = gend;
  const long long lo = a.row_start, hi = a.row_start + a.rows;
  l0 = (g0 > lo ? g0 : lo) - lo;
  l1 = (g1 < hi ? g1 : hi) - lo;
}

template <typename T, int VEC, int CPT, int RPI, int MAXR, bool RMS>
__global__ void __maxnreg__(MAXR) norm_fwd_kernel(const NormArgs a) {
  __shared__ __align__(16) float red[2][RPI * 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  for (int i = tid; i < 2 * RPI * 32; i += blockDim.x) (&red[0][0])[i] = 0.f;
  __syncthreads();

  const int H = a.hidden;
  const int nvec = H / VEC;
  const float inv_h = 1.f / static_cast<float>(H);
  const T* __restrict__ x = static_cast<const T*>(a.x);
  const T* __restrict__ scale = static_cast<const T*>(a.scale);
  const T* __restrict__ shift = static_cast<const T*>(a.shift);
  T* __restrict__ y = static_cast<T*>(a.y);
  int phase = 0;

  bool active[CPT];
  int col[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const int iv = tid + c * blockDim.x;
    active[c] = iv < nvec;
    col[c] = iv * VEC;
  }

  for (long long item = blockIdx.x; item < a.n_items; item += gridDim.x) {
    long long b, bi, l0, l1;
    item_rows(a, item, b, bi, l0, l1);
    if (l0 >= l1) continue;

    float sc[CPT][VEC], sh[CPT][VEC];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      Vec<T, VEC> vs, vh;
      vs.zero();
      vh.zero();
      if (active[c]) {
        vs.load(scale + b * H + col[c]);
        vh.load(shift + b * H + col[c]);
      }
      vs.unpack(sc[c]);
      vh.unpack(sh[c]);
#pragma unroll
      for (int k = 0; k < VEC; ++k) sc[c][k] += 1.f;
    }

    for (long long r0 = l0; r0 < l1; r0 += RPI) {
      Vec<T, VEC> xv[RPI][CPT];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          xv[j][c].zero();
          if (active[c] && r0 + j < l1) xv[j][c].load_stream(x + (r0 + j) * H + col[c]);
        }
      }

      float mean[RPI];
      if constexpr (!RMS) {
        float s[1][RPI];
#pragma unroll
        for (int j = 0; j < RPI; ++j) {
          float acc = 0.f;
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            float f[VEC];
            xv[j][c].unpack(f);
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc += f[k];
          }
          s[0][j] = acc;
        }
        cta_sum_rows<1, RPI>(s, red[phase], lane, warp, warps);
        phase ^= 1;
#pragma unroll
        for (int j = 0; j < RPI; ++j) mean[j] = s[0][j] * inv_h;
      } else {
#pragma unroll
        for (int j = 0; j < RPI; ++j) mean[j] = 0.f;
      }

      // second pass over the registers: sum of squared deviations (no E[x^2]-mean^2 cancellation)
      float q[1][RPI];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          if (active[c]) {
            float f[VEC];
            xv[j][c].opaque();
            xv[j][c].unpack(f);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
              const float d = f[k] - mean[j];
              acc = fmaf(d, d, acc);
            }
          }
        }
        q[0][j] = acc;
      }
      cta_sum_rows<1, RPI>(q, red[phase], lane, warp, warps);
      phase ^= 1;

      float rstd[RPI];
#pragma unroll
      for (int j = 0; j < RPI; ++j) rstd[j] = 1.f / sqrtf(q[0][j] * inv_h + a.eps);

#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        if (r0 + j < l1) {
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            if (active[c]) {
              float f[VEC];
              xv[j][c].opaque();
              xv[j][c].unpack(f);
#pragma unroll
              for (int k = 0; k < VEC; ++k)
                f[k] = fmaf((f[k] - mean[j]) * rstd[j], sc[c][k], sh[c][k]);
              Vec<T, VEC> out;
              out.pack(f);
              out.store(y + (r0 + j) * H + col[c]);
            }
          }
          if (tid == j && a.invstd != nullptr) {
            if constexpr (!RMS) a.mean[r0 + j] = mean[j];
            a.invstd[r0 + j] = rstd[j];
          }
        }
      }
    }
  }
}

template <typename T, int VEC, int CPT, int RPI, int MAXR, bool RMS, bool DX, bool DP>
__global__ void __maxnreg__(MAXR) norm_bwd_kernel(const NormArgs a) {
  constexpr int Q = RMS ? 1 : 2;  // row sums needed for dx: [sum dxhat,] sum dxhat*xhat
  __shared__ __align__(16) float red[2][Q * RPI * 32];
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  for (int i = tid; i < 2 * Q * RPI * 32; i += blockDim.x) (&red[0][0])[i] = 0.f;
  __syncthreads();

  const int H = a.hidden;
  const int nvec = H / VEC;
  const float inv_h = 1.f / static_cast<float>(H);
  const T* __restrict__ x = static_cast<const T*>(a.x);
  const T* __restrict__ dy = static_cast<const T*>(a.dy);
  const T* __restrict__ scale = static_cast<const T*>(a.scale);
  T* __restrict__ dx = static_cast<T*>(a.dx);
  int phase = 0;

  bool active[CPT];
  int col[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const int iv = tid + c * blockDim.x;
    active[c] = iv < nvec;
    col[c] = iv * VEC;
  }

  for (long long item = blockIdx.x; item < a.n_items; item += gridDim.x) {
    long long b, bi, l0, l1;
    item_rows(a, item, b, bi, l0, l1);
    // an item outside the shard still takes part in stage 2 (it contributes zeros)
    float sc1[CPT][VEC];
    float acc_s[CPT][VEC], acc_h[CPT][VEC];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      if constexpr (DX) {
        Vec<T, VEC> vs;
        vs.zero();
        if (active[c]) vs.load(scale + b * H + col[c]);
        vs.unpack(sc1[c]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) sc1[c][k] += 1.f;
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        acc_s[c][k] = 0.f;
        acc_h[c][k] = 0.f;
      }
    }

    for (long long r0 = l0; r0 < l1; r0 += RPI) {
      Vec<T, VEC> xv[RPI][CPT], gv[RPI][CPT];
      float rmean[RPI], rstd[RPI];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        const bool row_ok = r0 + j < l1;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          xv[j][c].zero();
          gv[j][c].zero();
          if (active[c] && row_ok) {
            gv[j][c].load_stream(dy + (r0 + j) * H + col[c]);
            xv[j][c].load_stream(x + (r0 + j) * H + col[c]);
          }
        }
        rstd[j] = row_ok ? __ldg(a.invstd + r0 + j) : 0.f;
        if constexpr (!RMS) {
          rmean[j] = row_ok ? __ldg(a.mean + r0 + j) : 0.f;
        } else {
          rmean[j] = 0.f;
        }
      }

      float p[Q][RPI];
      if constexpr (DX) {
#pragma unroll
        for (int j = 0; j < RPI; ++j) {
          float p0 = 0.f, p1 = 0.f;
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            float fx[VEC], fg[VEC];
            xv[j][c].unpack(fx);
            gv[j][c].unpack(fg);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
              const float xhat = (fx[k] - rmean[j]) * rstd[j];
              const float dxh = fg[k] * sc1[c][k];  // zero on inactive columns and rows
              p0 += dxh;
              p1 = fmaf(dxh, xhat, p1);
            }
          }
          if constexpr (!RMS) p[0][j] = p0;
          p[Q - 1][j] = p1;
        }
        cta_sum_rows<Q, RPI>(p, red[phase], lane, warp, warps);
        phase ^= 1;
      }

#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        if (r0 + j < l1) {
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            if (active[c]) {
              float fx[VEC], fg[VEC], out[VEC];
              if constexpr (DX) {
                xv[j][c].opaque();
                gv[j][c].opaque();
              }
              xv[j][c].unpack(fx);
              gv[j][c].unpack(fg);
#pragma unroll
              for (int k = 0; k < VEC; ++k) {
                const float xhat = (fx[k] - rmean[j]) * rstd[j];
                if constexpr (DX) {
                  const float dxh = fg[k] * sc1[c][k];
                  float t = dxh;
                  if constexpr (!RMS) t -= p[0][j] * inv_h;
                  t = fmaf(-xhat, p[Q - 1][j] * inv_h, t);
                  out[k] = rstd[j] * t;
                }
                if constexpr (DP) {
                  acc_h[c][k] += fg[k];
                  acc_s[c][k] = fmaf(fg[k], xhat, acc_s[c][k]);
                }
              }
              if constexpr (DX) {
                Vec<T, VEC> o;
                o.pack(out);
                o.store(dx + (r0 + j) * H + col[c]);
              }
            }
          }
        }
      }
    }

    if constexpr (DP) {
      constexpr int FV = (VEC % 4 == 0) ? 4 : 1;  // fp32 partials move as float4 when columns allow
      using FVec = Vec<float, FV>;
      const int T_ = a.tiles_per_sample;
      if (T_ == 1) {
        if (l0 < l1) {
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            if (active[c]) {
#pragma unroll
              for (int k = 0; k < VEC; k += FV) {
                FVec vs, vh;
#pragma unroll
                for (int e = 0; e < FV; ++e) {
                  vs.v[e] = acc_s[c][k + e];
                  vh.v[e] = acc_h[c][k + e];
                }
                vs.store(a.dscale + b * H + col[c] + k);
                vh.store(a.dshift + b * H + col[c] + k);
              }
            }
          }
        }
      } else {
        float* part = a.ws_part + item * 2 * H;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          if (active[c]) {
#pragma unroll
            for (int k = 0; k < VEC; k += FV) {
              FVec vs, vh;
#pragma unroll
              for (int e = 0; e < FV; ++e) {
                vs.v[e] = acc_s[c][k + e];
                vh.v[e] = acc_h[c][k + e];
              }
              vs.store(part + col[c] + k);
              vh.store(part + H + col[c] + k);
            }
          }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
          const unsigned int prev = atomicAdd(a.ws_cnt + bi, 1u);
          s_last = (prev == static_cast<unsigned int>(T_ - 1)) ? 1 : 0;
        }
        __syncthreads();
        if (s_last) {
          __threadfence();
          // stage 2: sum this sample's tile partials in tile order
          const float* base = a.ws_part + bi * T_ * 2 * H;
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            if (active[c]) {
#pragma unroll
              for (int k = 0; k < VEC; k += FV) {
                float ts[FV], th[FV];
#pragma unroll
                for (int e = 0; e < FV; ++e) ts[e] = th[e] = 0.f;
                for (int t = 0; t < T_; ++t) {
                  const float* ps = base + static_cast<long long>(t) * 2 * H + col[c] + k;
                  if constexpr (FV == 4) {
                    const float4 u = __ldcg(reinterpret_cast<const float4*>(ps));
                    const float4 w = __ldcg(reinterpret_cast<const float4*>(ps + H));
                    ts[0] += u.x; ts[1] += u.y; ts[2] += u.z; ts[3] += u.w;
                    th[0] += w.x; th[1] += w.y; th[2] += w.z; th[3] += w.w;
                  } else {
                    ts[0] += __ldcg(ps);
                    th[0] += __ldcg(ps + H);
                  }
                }
                FVec vs, vh;
#pragma unroll
                for (int e = 0; e < FV; ++e) {
                  vs.v[e] = ts[e];
                  vh.v[e] = th[e];
                }
                vs.store(a.dscale + b * H + col[c] + k);
                vh.store(a.dshift + b * H + col[c] + k);
              }
            }
          }
          if (tid == 0) a.ws_cnt[bi] = 0u;  // leave the counter ready for the next launch
        }
      }
    }
  }
}

// ------------------------------------------------------------------ launch
// RPIF / RPIB: rows in flight per thread in the forward / backward kernels; MAXRF / MAXRB: their
// register caps (threads x registers decides how many CTAs share an SM).
template <typename T, int VEC, int CPT, int RPIF, int MAXRF, int RPIB, int MAXRB>
static const void* pick_kernel(int mode, bool rms) {
  switch (mode) {
    case kFwd:
      return rms ? (const void*)norm_fwd_kernel<T, VEC, CPT, RPIF, MAXRF, true>
                 : (const void*)norm_fwd_kernel<T, VEC, CPT, RPIF, MAXRF, false>;
    case kBwdDx:
      return rms ? (const void*)norm_bwd_kernel<T, VEC, CPT, RPIB, MAXRB, true, true, false>
                 : (const void*)norm_bwd_kernel<T, VEC, CPT, RPIB, MAXRB, false, true, false>;
    case kBwdDparam:
      return rms ? (const void*)norm_bwd_kernel<T, VEC, CPT, RPIB, MAXRB, true, false, true>
                 : (const void*)norm_bwd_kernel<T, VEC, CPT, RPIB, MAXRB, false, false, true>;
    default:
      return rms ? (const void*)norm_bwd_kernel<T, VEC, CPT, RPIB, MAXRB, true, true, true>
                 : (const void*)norm_bwd_kernel<T, VEC, CPT, RPIB, MAXRB, false, true, true>;
  }
}

// Tile plan shared by the workspace-size query and the launcher.
struct TilePlan {
  long long b_first, n_samples;
  int tile_rows, tiles_per_sample;
  long long n_items;
};
TilePlan plan_tiles(long long rows, long long row_start, long long seq_len, int tile_rows);
int tile_rows_override();  // > 0 when a tuning override is set

template <typename T, int VEC>
int launch_norm_vec(NormArgs a, cudaStream_t st) {
  const int nvec = a.hidden / VEC;
  const void* fn = nullptr;
  int nt = 0;
  if (nvec <= 256) {
    fn = pick_kernel<T, VEC, 1, 8, 96, 4, 128>(a.mode, a.rms);
    nt = (nvec + 31) / 32 * 32;
  } else if (nvec <= 512) {
    fn = pick_kernel<T, VEC, 1, 4, 64, 4, 128>(a.mode, a.rms);
    nt = (nvec + 31) / 32 * 32;
  } else if (nvec <= 1024) {
    fn = pick_kernel<T, VEC, 1, 4, 64, 2, 64>(a.mode, a.rms);
    nt = (nvec + 31) / 32 * 32;
  } else if (nvec <= 4096) {
    fn = pick_kernel<T, VEC, 4, 1, 64, 1, 64>(a.mode, a.rms);
    nt = ((nvec + 3) / 4 + 31) / 32 * 32;
  } else {
    return ND_ERR_UNSUPPORTED;
  }

  // Choose the tile height so that all items fit in one wave of resident CTAs
  // when the problem is small enough; otherwise use tall tiles and let the
  // persistent loop spread many items per CTA.
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, nt, 0) != cudaSuccess || occ < 1) {
    (void)cudaGetLastError();
    occ = 1;
  }
  const long long slots = static_cast<long long>(occ) * sm_count();
  TilePlan plan{};
  const int forced = tile_rows_override();
  if (forced > 0) {
    plan = plan_tiles(a.rows, a.row_start, a.seq_len, forced);
  } else {
    for (int k = 1; k <= 8; ++k) {
      plan = plan_tiles(a.rows, a.row_start, a.seq_len, 8 * k);
      if (plan.n_items <= slots) break;
    }
  }
  a.b_first = plan.b_first;
  a.n_samples = plan.n_samples;
  a.tile_rows = plan.tile_rows;
  a.tiles_per_sample = plan.tiles_per_sample;
  a.n_items = plan.n_items;
  if (a.n_items == 0) return ND_OK;
  const long long grid = a.n_items < slots ? a.n_items : slots;
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
int launch_norm(const NormArgs& a, cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(T);
  bool vec_ok = (a.hidden % VMAX) == 0;
  const void* ptrs[] = {a.x, a.scale, a.shift, a.y, a.dy, a.dx, a.dscale, a.dshift, a.ws_part};
  for (const void* p : ptrs) vec_ok = vec_ok && aligned16(p);
  return vec_ok ? launch_norm_vec<T, VMAX>(a, st) : launch_norm_vec<T, 1>(a, st);
}

}  // namespace nd
