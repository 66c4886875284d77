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
// backward pass writes one fp32 partial [2, H] per item (stage 1) and a second
// small kernel sums each sample's partials in index order (stage 2):
// deterministic, no atomics at all.
#pragma once

#include "common.cuh"
#include "ptx.cuh"

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
  float* ws_part;  // [slots][2][hidden] fp32 partial column sums (stage 1 of the dparam reduction)
  long long rows, row_start;
  int seq_len, hidden;
  float eps;
  int tile_rows, tiles_per_sample;
  long long b_first, n_samples, n_items;
  int mode;
  bool rms;
  int n_chunks;  // bulk-copy kernels: the shard's rows are split evenly into this many chunks, one per CTA
  long long chunk_base;  // rows / n_chunks
  int chunk_rem;         // rows % n_chunks
  int chunks_per_sample;  // > 0: the shard is whole samples and every sample is cut into this many chunks (no chunk
                          // crosses a sample boundary); 0: the shard's rows are cut evenly, whatever the samples
  int stages;    // shared-memory pipeline depth of the bulk-copy kernels
  int* err;    // device error word (set when a bounded wait expires)
  // forward with e4m3 output (warp-per-row kernel only): y holds bytes, q = saturate_e4m3(value / *q_scale),
  // *q_amax = max(*q_amax, max |value|) (nullable)
  const float* q_scale;
  float* q_amax;
  // forward with the gated residual in front (bulk-copy kernels only): x_new = x + gate[b] * branch is written to dx
  // and normalised; `dy` holds branch, `gate` the [B, H] gate (null: plain x + branch), `res` switches it on
  const void* gate;
  bool res;
  // bounded waits of the bulk-copy kernels: the limit (1 s unless a test shortens it) and a test switch that makes
  // CTA 0 leave its first copy unsent, so that its first wait runs out with nothing in flight
  unsigned long long wait_limit_ns;
  int withhold_first_copy;
};

// first row (local to the shard) of chunk c
// (chunks differ in size by at most one row: the first `chunk_rem` chunks hold `chunk_base` + 1 rows)
__device__ __host__ __forceinline__ long long chunk_start(long long chunk_base, int chunk_rem, long long c) {
  return c * chunk_base + (c < chunk_rem ? c : chunk_rem);
}

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
  griddep_launch_dependents();
  __syncthreads();
  griddep_wait();

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
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  for (int i = tid; i < 2 * Q * RPI * 32; i += blockDim.x) (&red[0][0])[i] = 0.f;
  griddep_launch_dependents();
  __syncthreads();
  griddep_wait();

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
      // stage 1 of the dparam reduction: this item's fp32 column sums go to its own slot of the
      // workspace (zeros if the item lies outside the shard); a second kernel sums each sample's
      // slots in index order.
      constexpr int FV = (VEC % 4 == 0) ? 4 : 1;  // fp32 partials move as float4 when columns allow
      using FVec = Vec<float, FV>;
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
    }
  }
}

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
int norm_variant();        // tuning: 0 = bulk-copy kernels where they apply, 1 = generic kernels everywhere
int launch_dparam_stage2(const NormArgs& a, cudaStream_t st);  // fixed-order sum of the stage-1 partials
constexpr int kMaxChunksPerSm = 8;  // upper bound on resident CTAs per SM used to size the workspace

}  // namespace nd
