// AdaLN / AdaRMSNorm kernels with a bulk-copy (TMA) pipeline into shared memory (sm_100a).
//
// Work split. The shard's rows are cut into `n_chunks` contiguous chunks, one per CTA and at most
// one CTA per resident slot, so a launch is a single wave whatever the batch and sequence sizes
// are: `chunks_per_sample` equal chunks of every sample when the shard is whole samples and that
// fills the slots (no chunk crosses a sample boundary then), equal chunks of the shard's rows
// otherwise. Inside its chunk a CTA walks groups of up to RPI rows that never cross a sample
// boundary (the modulation vector and the dscale/dshift column sums are per sample).
//
// Data path. The rows of a group are contiguous in global memory, so ONE cp.async.bulk per
// input tensor lands a whole group in a shared-memory stage. Thread 0 keeps `stages` groups in
// flight ahead of the consumers: the bytes in flight per SM are set by shared memory (up to
// ~220 KB), not by registers. All threads wait on the stage's mbarrier, turn their 16-byte
// column vector of each row into packed fp32 once, and compute; a stage is refilled right
// after the CTA-wide barrier that follows its last read, so no "empty" barriers exist. Every
// mbarrier wait is bounded (1 s): on expiry the device error word is set and the whole CTA
// leaves together.
//
// dparam. Each (chunk, sample) segment writes its fp32 column sums to workspace slot
// chunk + (sample - first sample of the shard); slots of one sample are consecutive, and a second
// small kernel sums them in index order. No atomics, no fences, deterministic.
#pragma once

#include <type_traits>

#include "norm_rowmath.cuh"
#include "ptx.cuh"

namespace nd {

constexpr int kMaxStages = 16;
constexpr int kBarrierBytes = 128;  // kMaxStages mbarriers at the head of dynamic shared memory

// Walks the row groups of one chunk: groups of up to `rpi` rows that stay inside one sample.
struct GroupCursor {
  long long r, r_end;   // next row, end of the chunk (local to the shard)
  long long b, s_end;   // sample of row r, end of that sample clipped to the chunk (local)
  __device__ __forceinline__ bool init(const NormArgs& a) {
    if (a.chunks_per_sample > 0) {  // chunk j of sample bi: the sample's rows cut evenly
      const long long k = a.chunks_per_sample;
      const long long bi = blockIdx.x / k, j = blockIdx.x - bi * k;
      const long long base = a.seq_len / k, rem = a.seq_len - base * k;
      r = bi * a.seq_len + j * base + (j < rem ? j : rem);
      r_end = r + base + (j < rem ? 1 : 0);
      b = a.b_first + bi;
      clip_sample(a);
      return r < r_end;
    }
    r = chunk_start(a.chunk_base, a.chunk_rem, blockIdx.x);
    r_end = chunk_start(a.chunk_base, a.chunk_rem, blockIdx.x + 1);
    if (r >= r_end) return false;
    const unsigned long long g = static_cast<unsigned long long>(a.row_start + r);
    // the only division of the walk; 32-bit when the global row index allows
    b = (g >> 32) == 0 ? static_cast<long long>(static_cast<unsigned int>(g) / static_cast<unsigned int>(a.seq_len))
                       : static_cast<long long>(g / static_cast<unsigned long long>(a.seq_len));
    clip_sample(a);
    return true;
  }
  __device__ __forceinline__ void clip_sample(const NormArgs& a) {
    const long long e = (b + 1) * a.seq_len - a.row_start;
    s_end = e < r_end ? e : r_end;
  }
  __device__ __forceinline__ int group_rows(int rpi) const {
    const long long left = s_end - r;
    return left < rpi ? static_cast<int>(left) : rpi;
  }
  // advance past the current group; false at the end of the chunk
  __device__ __forceinline__ bool next(const NormArgs& a, int rpi) {
    r += group_rows(rpi);
    if (r >= r_end) return false;
    if (r == s_end) {  // the next sample starts here
      ++b;
      clip_sample(a);
    }
    return true;
  }
};

// Issue the bulk copies of the group under `pc` into stage `s` (called by one thread).
template <typename T, int RPI, bool TWO>
__device__ __forceinline__ void issue_group(const NormArgs& a, const GroupCursor& pc, int s, uint64_t* full,
                                            unsigned char* buf, uint32_t row_bytes) {
  const uint32_t bytes = static_cast<uint32_t>(pc.group_rows(RPI)) * row_bytes;
  const uint32_t stage_total = (TWO ? 2u : 1u) * RPI * row_bytes;
  unsigned char* dst = buf + static_cast<size_t>(s) * stage_total;
  const long long off = pc.r * a.hidden;
  mbar_expect_tx(&full[s], TWO ? 2 * bytes : bytes);
  bulk_load_1d(dst, static_cast<const T*>(a.x) + off, bytes, &full[s]);
  if constexpr (TWO) bulk_load_1d(dst + RPI * row_bytes, static_cast<const T*>(a.dy) + off, bytes, &full[s]);
}

// Common prologue: barriers, producer cursor, first `stages` groups in flight.
template <typename T, int RPI, bool TWO>
__device__ __forceinline__ void pipeline_start(const NormArgs& a, uint64_t* full, unsigned char* buf,
                                               uint32_t row_bytes, GroupCursor& pc, bool& pc_valid) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  griddep_launch_dependents();
  __syncthreads();
  griddep_wait();  // nothing above reads global memory; everything below may
  pc_valid = false;
  if (threadIdx.x == 0) {
    pc_valid = pc.init(a);
    for (int s = 0; s < a.stages && pc_valid; ++s) {
      // test switch: CTA 0 never sends its first group, so the wait on stage 0 expires with nothing in flight
      if (!(a.withhold_first_copy && blockIdx.x == 0 && s == 0)) issue_group<T, RPI, TWO>(a, pc, s, full, buf, row_bytes);
      pc_valid = pc.next(a, RPI);
    }
  }
}

// A CTA whose wait expired lets copies that may still be in flight land before it exits.
__device__ __forceinline__ void drain_after_abort() {
  const unsigned long long t0 = global_ns();
  while (global_ns() - t0 < 200000ull) __nanosleep(1000);
}

// RES: the input of the normalisation is the gated residual x + gate[b] * branch (gate null: x + branch), which is
// written out as well (a.dx = x_new; a.dy = branch): one pass instead of a residual kernel followed by a norm
// kernel. The sum is rounded to T first and the statistics are taken of the ROUNDED values, so that y, mean and
// 1/std are exactly what the norm of the stored x_new gives.
template <typename T, int VEC, int RPI, int MAXR, bool RMS, bool RES = false>
__global__ void __maxnreg__(MAXR) norm_fwd_tma(const NormArgs a) {
  constexpr int NP = VEC / 2;
  extern __shared__ __align__(128) unsigned char dsm[];
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm);
  unsigned char* buf = dsm + kBarrierBytes;
  __shared__ __align__(16) float red[2][RPI * 32];
  __shared__ __align__(16) float zero16[4];  // what idle lanes of the last warp read instead of a column
  __shared__ int s_abort;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  if (tid < 4) zero16[tid] = 0.f;
  if (tid == 0) s_abort = 0;

  const int H = a.hidden;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const uint32_t stage_total = (RES ? 2 : 1) * RPI * row_bytes;  // x rows [then branch rows]
  const bool active = tid < H / VEC;
  const int col = active ? tid * VEC : 0;
  const uint32_t src_stride = active ? row_bytes : 0u;
  const uint32_t br_off = active ? RPI * row_bytes : 0u;
  const float inv_h = 1.f / static_cast<float>(H);
  const float eps = a.eps;
  const long long row_elems = H;
  int phase = 0;

  GroupCursor pc;
  bool pc_valid;
  pipeline_start<T, RPI, RES>(a, full, buf, row_bytes, pc, pc_valid);

  int stage = 0;
  uint32_t parity = 0;
  GroupCursor cc;
  bool more = cc.init(a);
  while (more) {
    // per-segment setup: modulation vector of the sample, in registers
    const long long b = cc.b;
    float2 sc[NP], sh[NP];
    {
      Vec<T, VEC> vs, vh;
      vs.load(static_cast<const T*>(a.scale) + b * H + col);
      vh.load(static_cast<const T*>(a.shift) + b * H + col);
      unpack2<T, VEC>(vs, sc);
      unpack2<T, VEC>(vh, sh);
#pragma unroll
      for (int i = 0; i < NP; ++i) sc[i] = __fadd2_rn(sc[i], make_float2(1.f, 1.f));
    }
    [[maybe_unused]] float2 gt[NP];
    if constexpr (RES) {
#pragma unroll
      for (int i = 0; i < NP; ++i) gt[i] = make_float2(1.f, 1.f);
      if (a.gate != nullptr) {
        Vec<T, VEC> vg;
        vg.load(static_cast<const T*>(a.gate) + b * H + col);
        unpack2<T, VEC>(vg, gt);
      }
    }
    do {
      const long long r = cc.r;
      const int nrows = cc.group_rows(RPI);
      // A wait that expires raises the CTA's abort flag; everybody sees it after the next barrier (the
      // one inside the row reduction) and the CTA leaves together.
      if (!mbar_wait_1s(&full[stage], parity, a.err, 1, a.wait_limit_ns)) s_abort = 1;
      // this thread's 16-byte column of each row (rows past the group's end hold stale data: they are
      // reduced like the others, independently per row, and never stored)
      const unsigned char* src =
          active ? buf + static_cast<size_t>(stage) * stage_total + col * sizeof(T) : reinterpret_cast<const unsigned char*>(zero16);
      float2 X[RPI][NP];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        Vec<T, VEC> pk;
        *reinterpret_cast<uint4*>(pk.v) = *reinterpret_cast<const uint4*>(src + j * src_stride);
        unpack2<T, VEC>(pk, X[j]);
        if constexpr (RES) {
          Vec<T, VEC> pb;
          *reinterpret_cast<uint4*>(pb.v) = *reinterpret_cast<const uint4*>(src + br_off + j * src_stride);
          float2 Bv[NP];
          unpack2<T, VEC>(pb, Bv);
#pragma unroll
          for (int i = 0; i < NP; ++i) X[j][i] = __ffma2_rn(gt[i], Bv[i], X[j][i]);
          pack2<T, VEC>(X[j], pk);  // the one rounding of the residual stream
          if (active && j < nrows) pk.store(static_cast<T*>(a.dx) + (r + j) * row_elems + col);
          unpack2<T, VEC>(pk, X[j]);  // the norm sees what was stored
        }
      }

      float mean_mine[1] = {0.f};
      bool refilled = false;
      if constexpr (!RMS) {
        float s[1][RPI];
#pragma unroll
        for (int j = 0; j < RPI; ++j) {
          float2 acc = X[j][0];
#pragma unroll
          for (int i = 1; i < NP; ++i) acc = __fadd2_rn(acc, X[j][i]);
          s[0][j] = acc.x + acc.y;
        }
        cta_sum_rows_post<1, RPI>(s, mean_mine, red[phase], lane, warp, warps,
                                  [&](int, float t) { return -t * inv_h; });  // broadcast -mean
        phase ^= 1;
        if (*static_cast<volatile int*>(&s_abort)) {
          drain_after_abort();
          return;
        }
        if (tid == 0 && pc_valid) {  // every thread has read the stage: refill it
          fence_proxy_async_smem();
          issue_group<T, RPI, RES>(a, pc, stage, full, buf, row_bytes);
          pc_valid = pc.next(a, RPI);
        }
        refilled = true;
#pragma unroll
        for (int j = 0; j < RPI; ++j) {
          const float2 nm = make_float2(s[0][j], s[0][j]);
#pragma unroll
          for (int i = 0; i < NP; ++i) X[j][i] = __fadd2_rn(X[j][i], nm);  // deviations, in place
        }
      }

      float q[1][RPI], rstd_mine[1];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        float2 acc = __fmul2_rn(X[j][0], X[j][0]);
#pragma unroll
        for (int i = 1; i < NP; ++i) acc = __ffma2_rn(X[j][i], X[j][i], acc);
        q[0][j] = active ? acc.x + acc.y : 0.f;  // an idle lane's deviations are -mean, not 0
      }
      cta_sum_rows_post<1, RPI>(q, rstd_mine, red[phase], lane, warp, warps,
                                [&](int, float t) { return rsqrt_newton(fmaf(t, inv_h, eps)); });  // broadcast 1/std
      phase ^= 1;
      if (*static_cast<volatile int*>(&s_abort)) {
        drain_after_abort();
        return;
      }
      if (!refilled && tid == 0 && pc_valid) {
        fence_proxy_async_smem();
        issue_group<T, RPI, RES>(a, pc, stage, full, buf, row_bytes);
        pc_valid = pc.next(a, RPI);
      }

      if (tid < RPI && tid < nrows && a.invstd != nullptr) {  // lane j of warp 0 owns row j's statistics
        if constexpr (!RMS) a.mean[r + tid] = -mean_mine[0];
        a.invstd[r + tid] = rstd_mine[0];
      }
      if (active) {
        T* yp = static_cast<T*>(a.y) + r * row_elems + col;
        const int limit = nrows == RPI ? RPI : nrows;  // a full group stores without per-row tests
#pragma unroll
        for (int j = 0; j < RPI; ++j) {
          if (nrows == RPI || j < limit) {
            const float2 r2 = make_float2(q[0][j], q[0][j]);
            float2 out[NP];
#pragma unroll
            for (int i = 0; i < NP; ++i) out[i] = __ffma2_rn(__fmul2_rn(X[j][i], r2), sc[i], sh[i]);
            Vec<T, VEC> o;
            pack2<T, VEC>(out, o);
            o.store(yp);
          }
          yp += row_elems;
        }
      }
      if (++stage == a.stages) {
        stage = 0;
        parity ^= 1u;
      }
      more = cc.next(a, RPI);
    } while (more && cc.b == b);
  }
}

template <typename T, int VEC, int RPI, int MAXR, bool RMS, bool DX, bool DP>
__global__ void __maxnreg__(MAXR) norm_bwd_tma(const NormArgs a) {
  constexpr int NP = VEC / 2;
  constexpr int Q = RMS ? 1 : 2;  // row sums needed for dx: [sum dxhat,] sum dxhat*xhat
  extern __shared__ __align__(128) unsigned char dsm[];
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm);
  unsigned char* buf = dsm + kBarrierBytes;
  __shared__ __align__(16) float red[2][Q * RPI * 32];
  __shared__ __align__(16) float zero16[4];
  __shared__ int s_abort;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  if (tid < 4) zero16[tid] = 0.f;
  if (tid == 0) s_abort = 0;

  const int H = a.hidden;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const uint32_t stage_total = 2 * RPI * row_bytes;  // x rows then dy rows
  const bool active = tid < H / VEC;
  const int col = active ? tid * VEC : 0;
  const uint32_t src_stride = active ? row_bytes : 0u;
  const uint32_t dy_off = active ? RPI * row_bytes : 0u;
  const float inv_h = 1.f / static_cast<float>(H);
  const long long row_elems = H;
  int phase = 0;

  GroupCursor pc;
  bool pc_valid;
  pipeline_start<T, RPI, true>(a, full, buf, row_bytes, pc, pc_valid);
  int stage = 0;
  uint32_t parity = 0;

  GroupCursor cc;
  bool more = cc.init(a);
  while (more) {
    // one segment = the rows of one sample inside this chunk
    const long long b = cc.b;
    float2 sc1[NP], acc_s[NP], acc_h[NP];
#pragma unroll
    for (int i = 0; i < NP; ++i) acc_s[i] = acc_h[i] = make_float2(0.f, 0.f);
    if constexpr (DX) {
      Vec<T, VEC> vs;
      vs.load(static_cast<const T*>(a.scale) + b * H + col);
      unpack2<T, VEC>(vs, sc1);
#pragma unroll
      for (int i = 0; i < NP; ++i) sc1[i] = __fadd2_rn(sc1[i], make_float2(1.f, 1.f));
    }

    do {
      const long long r = cc.r;
      const int nrows = cc.group_rows(RPI);
      const bool full_group = nrows == RPI;
      float rstd[RPI], nmean[RPI];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        const long long rr = r + (full_group || j < nrows ? j : nrows - 1);  // clamped inside the group
        rstd[j] = __ldg(a.invstd + rr);
        if constexpr (!RMS) nmean[j] = -__ldg(a.mean + rr);
        else nmean[j] = 0.f;
      }
      if (!mbar_wait_1s(&full[stage], parity, a.err, 2, a.wait_limit_ns)) s_abort = 1;  // seen by all after the next barrier
      const unsigned char* src =
          active ? buf + static_cast<size_t>(stage) * stage_total + col * sizeof(T) : reinterpret_cast<const unsigned char*>(zero16);
      float2 X[RPI][NP], G[RPI][NP];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        Vec<T, VEC> px, pg;
        *reinterpret_cast<uint4*>(px.v) = *reinterpret_cast<const uint4*>(src + j * src_stride);
        *reinterpret_cast<uint4*>(pg.v) = *reinterpret_cast<const uint4*>(src + dy_off + j * src_stride);
        unpack2<T, VEC>(px, X[j]);
        unpack2<T, VEC>(pg, G[j]);
      }
      if (!full_group) {  // rows past the group's end hold stale data: keep them out of the column sums
#pragma unroll
        for (int j = 0; j < RPI; ++j) {
          if (j >= nrows) {
#pragma unroll
            for (int i = 0; i < NP; ++i) {
              G[j][i] = make_float2(0.f, 0.f);
              X[j][i] = make_float2(0.f, 0.f);
            }
          }
        }
      }

      float p[Q][RPI];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        const float2 r2 = make_float2(rstd[j], rstd[j]), m2 = make_float2(nmean[j], nmean[j]);
        float2 p0 = make_float2(0.f, 0.f), p1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < NP; ++i) {
          // xhat = (x - mean) * rstd in place (idle lanes read zeros: dy = 0 makes every product 0)
          if constexpr (!RMS) X[j][i] = __fadd2_rn(X[j][i], m2);
          X[j][i] = __fmul2_rn(X[j][i], r2);
          if constexpr (DP) {
            acc_h[i] = __fadd2_rn(acc_h[i], G[j][i]);
            acc_s[i] = __ffma2_rn(G[j][i], X[j][i], acc_s[i]);
          }
          if constexpr (DX) {
            G[j][i] = __fmul2_rn(G[j][i], sc1[i]);  // dxhat in place
            if constexpr (!RMS) p0 = __fadd2_rn(p0, G[j][i]);
            p1 = __ffma2_rn(G[j][i], X[j][i], p1);
          }
        }
        if constexpr (DX) {
          if constexpr (!RMS) p[0][j] = p0.x + p0.y;
          p[Q - 1][j] = p1.x + p1.y;
        }
      }
      if constexpr (DX) {
        float mine[Q];
        cta_sum_rows_post<Q, RPI>(p, mine, red[phase], lane, warp, warps,
                                  [&](int, float t) { return -t * inv_h; });  // broadcast -mean_h(.)
        phase ^= 1;
      } else {
        __syncthreads();  // every thread has read the stage
      }
      if (*static_cast<volatile int*>(&s_abort)) {
        drain_after_abort();
        return;
      }
      if (tid == 0 && pc_valid) {
        fence_proxy_async_smem();
        issue_group<T, RPI, true>(a, pc, stage, full, buf, row_bytes);
        pc_valid = pc.next(a, RPI);
      }
      if (++stage == a.stages) {
        stage = 0;
        parity ^= 1u;
      }
      if constexpr (DX) {
        if (active) {
          T* dp = static_cast<T*>(a.dx) + r * row_elems + col;
#pragma unroll
          for (int j = 0; j < RPI; ++j) {
            if (full_group || j < nrows) {
              const float2 c2v = make_float2(p[Q - 1][j], p[Q - 1][j]), r2 = make_float2(rstd[j], rstd[j]);
              float2 out[NP];
#pragma unroll
              for (int i = 0; i < NP; ++i) {
                float2 t = G[j][i];
                if constexpr (!RMS) t = __fadd2_rn(t, make_float2(p[0][j], p[0][j]));
                t = __ffma2_rn(X[j][i], c2v, t);
                out[i] = __fmul2_rn(t, r2);
              }
              Vec<T, VEC> o;
              pack2<T, VEC>(out, o);
              o.store(dp);
            }
            dp += row_elems;
          }
        }
      }
      more = cc.next(a, RPI);
    } while (more && cc.b == b);

    if constexpr (DP) {
      // stage 1 of the dparam reduction: this segment's column sums go to their own workspace slot
      if (active) {
        constexpr int NF4 = VEC / 4;  // float4 chunks per thread (VEC is 4 or 8)
        float* part = a.ws_part + (static_cast<long long>(blockIdx.x) + (b - a.b_first)) * 2 * H + col;
#pragma unroll
        for (int k = 0; k < NF4; ++k) {
          reinterpret_cast<float4*>(part)[k] = make_float4(acc_s[2 * k].x, acc_s[2 * k].y, acc_s[2 * k + 1].x, acc_s[2 * k + 1].y);
          reinterpret_cast<float4*>(part + H)[k] = make_float4(acc_h[2 * k].x, acc_h[2 * k].y, acc_h[2 * k + 1].x, acc_h[2 * k + 1].y);
        }
      }
    }
  }
}

// The forward with the flat walk of norm_bwd_tma_flat (below): every chunk lies inside one sample, so the modulation
// vectors are loaded once, positions are 32-bit offsets from bases computed once, and full groups run without row
// predicates. Same arithmetic in the same order as norm_fwd_tma: bit-identical results.
template <typename T, int VEC, int RPI, int MAXR, bool RMS, bool RES = false>
__global__ void __maxnreg__(MAXR) norm_fwd_tma_flat(const NormArgs a) {
  constexpr int NP = VEC / 2;
  extern __shared__ __align__(128) unsigned char dsm[];
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm);
  unsigned char* buf = dsm + kBarrierBytes;
  __shared__ __align__(16) float red[2][RPI * 32];
  __shared__ __align__(16) float zero16[4];  // what idle lanes of the last warp read instead of a column
  __shared__ int s_abort;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  if (tid < 4) zero16[tid] = 0.f;
  if (tid == 0) s_abort = 0;

  const int H = a.hidden;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const uint32_t stage_total = (RES ? 2 : 1) * RPI * row_bytes;  // x rows [then branch rows]
  const bool active = tid < H / VEC;
  const int col = active ? tid * VEC : 0;
  const uint32_t src_stride = active ? row_bytes : 0u;
  [[maybe_unused]] const uint32_t br_off = active ? RPI * row_bytes : 0u;
  const float inv_h = 1.f / static_cast<float>(H);
  const float eps = a.eps;

  // this CTA's chunk: rows [r0, r0 + n) of sample bi of the shard (whole samples, cut evenly)
  const int k = a.chunks_per_sample, seq = static_cast<int>(a.seq_len);
  const int bi = static_cast<int>(blockIdx.x) / k, cj = static_cast<int>(blockIdx.x) - bi * k;
  const int cbase = seq / k, crem = seq - cbase * k;
  const long long r0 = static_cast<long long>(bi) * seq + cj * cbase + (cj < crem ? cj : crem);
  const int n = cbase + (cj < crem ? 1 : 0);
  const int n_groups = (n + RPI - 1) / RPI;
  const long long b = a.b_first + bi;

  if (tid == 0) {
    for (int s = 0; s < a.stages; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  griddep_launch_dependents();
  __syncthreads();
  griddep_wait();  // nothing above reads global memory; everything below may

  const T* xg = static_cast<const T*>(a.x) + r0 * H;
  [[maybe_unused]] const T* bg = RES ? static_cast<const T*>(a.dy) + r0 * H : nullptr;
  int pg = 0;  // next group to request (thread 0 only)
  auto request = [&](int g, int s) {
    const int rows = n - g * RPI < RPI ? n - g * RPI : RPI;
    const uint32_t bytes = static_cast<uint32_t>(rows) * row_bytes;
    unsigned char* dst = buf + static_cast<uint32_t>(s) * stage_total;
    const size_t off = static_cast<size_t>(g) * RPI * H;
    mbar_expect_tx(&full[s], RES ? 2 * bytes : bytes);
    bulk_load_1d(dst, xg + off, bytes, &full[s]);
    if constexpr (RES) bulk_load_1d(dst + RPI * row_bytes, bg + off, bytes, &full[s]);
  };
  if (tid == 0) {
    for (int s = 0; s < a.stages && pg < n_groups; ++s, ++pg) {
      // test switch: CTA 0 never sends its first group, so the wait on stage 0 expires with nothing in flight
      if (!(a.withhold_first_copy && blockIdx.x == 0 && s == 0)) request(pg, s);
    }
  }

  // the sample's modulation vector, in registers
  float2 sc[NP], sh[NP];
  {
    Vec<T, VEC> vs, vh;
    vs.load(static_cast<const T*>(a.scale) + b * H + col);
    vh.load(static_cast<const T*>(a.shift) + b * H + col);
    unpack2<T, VEC>(vs, sc);
    unpack2<T, VEC>(vh, sh);
#pragma unroll
    for (int i = 0; i < NP; ++i) sc[i] = __fadd2_rn(sc[i], make_float2(1.f, 1.f));
  }
  [[maybe_unused]] float2 gt[NP];
  if constexpr (RES) {
#pragma unroll
    for (int i = 0; i < NP; ++i) gt[i] = make_float2(1.f, 1.f);
    if (a.gate != nullptr) {
      Vec<T, VEC> vg;
      vg.load(static_cast<const T*>(a.gate) + b * H + col);
      unpack2<T, VEC>(vg, gt);
    }
  }
  T* yp = static_cast<T*>(a.y) + r0 * H + col;
  [[maybe_unused]] T* xn = RES ? static_cast<T*>(a.dx) + r0 * H + col : nullptr;
  float* mean_p = (!RMS && a.invstd != nullptr) ? a.mean + r0 : nullptr;
  float* inv_p = a.invstd != nullptr ? a.invstd + r0 : nullptr;
  const size_t group_elems = static_cast<size_t>(RPI) * H;
  int stage = 0, phase = 0;
  uint32_t parity = 0;

  auto refill = [&]() {
    if (tid == 0 && pg < n_groups) {  // every thread has read the stage: refill it
      fence_proxy_async_smem();
      request(pg, stage);
      ++pg;
    }
  };

  // one group of rows; FULL: all RPI rows exist (no row predicates). Returns false when the CTA must leave.
  auto group = [&](auto full_tag, int nrows) -> bool {
    constexpr bool FULL = decltype(full_tag)::value;
    // A wait that expires raises the CTA's abort flag; everybody sees it after the next barrier (the one inside
    // the row reduction) and the CTA leaves together.
    if (!mbar_wait_1s(&full[stage], parity, a.err, 1, a.wait_limit_ns)) s_abort = 1;
    // this thread's 16-byte column of each row (rows past the group's end hold stale data: they are reduced like
    // the others, independently per row, and never stored)
    const unsigned char* src =
        active ? buf + static_cast<uint32_t>(stage) * stage_total + col * sizeof(T) : reinterpret_cast<const unsigned char*>(zero16);
    float2 X[RPI][NP];
#pragma unroll
    for (int j = 0; j < RPI; ++j) {
      Vec<T, VEC> pk;
      *reinterpret_cast<uint4*>(pk.v) = *reinterpret_cast<const uint4*>(src + j * src_stride);
      unpack2<T, VEC>(pk, X[j]);
      if constexpr (RES) {
        Vec<T, VEC> pb;
        *reinterpret_cast<uint4*>(pb.v) = *reinterpret_cast<const uint4*>(src + br_off + j * src_stride);
        float2 Bv[NP];
        unpack2<T, VEC>(pb, Bv);
#pragma unroll
        for (int i = 0; i < NP; ++i) X[j][i] = __ffma2_rn(gt[i], Bv[i], X[j][i]);
        pack2<T, VEC>(X[j], pk);  // the one rounding of the residual stream
        if (active && (FULL || j < nrows)) pk.store(xn + static_cast<size_t>(j) * H);
        unpack2<T, VEC>(pk, X[j]);  // the norm sees what was stored
      }
    }

    float mean_mine[1] = {0.f};
    if constexpr (!RMS) {
      float s[1][RPI];
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        float2 acc = X[j][0];
#pragma unroll
        for (int i = 1; i < NP; ++i) acc = __fadd2_rn(acc, X[j][i]);
        s[0][j] = acc.x + acc.y;
      }
      cta_sum_rows_post<1, RPI>(s, mean_mine, red[phase], lane, warp, warps,
                                [&](int, float t) { return -t * inv_h; });  // broadcast -mean
      phase ^= 1;
      if (*static_cast<volatile int*>(&s_abort)) return false;
      refill();
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        const float2 nm = make_float2(s[0][j], s[0][j]);
#pragma unroll
        for (int i = 0; i < NP; ++i) X[j][i] = __fadd2_rn(X[j][i], nm);  // deviations, in place
      }
    }

    float q[1][RPI], rstd_mine[1];
#pragma unroll
    for (int j = 0; j < RPI; ++j) {
      float2 acc = __fmul2_rn(X[j][0], X[j][0]);
#pragma unroll
      for (int i = 1; i < NP; ++i) acc = __ffma2_rn(X[j][i], X[j][i], acc);
      q[0][j] = active ? acc.x + acc.y : 0.f;  // an idle lane's deviations are -mean, not 0
    }
    cta_sum_rows_post<1, RPI>(q, rstd_mine, red[phase], lane, warp, warps,
                              [&](int, float t) { return rsqrt_newton(fmaf(t, inv_h, eps)); });  // broadcast 1/std
    phase ^= 1;
    if (*static_cast<volatile int*>(&s_abort)) return false;
    if constexpr (RMS) refill();

    if (tid < RPI && (FULL || tid < nrows) && inv_p != nullptr) {  // lane j of warp 0 owns row j's statistics
      if constexpr (!RMS) mean_p[tid] = -mean_mine[0];
      inv_p[tid] = rstd_mine[0];
    }
    if (active) {
      T* out_p = yp;
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        if (FULL || j < nrows) {
          const float2 r2 = make_float2(q[0][j], q[0][j]);
          float2 out[NP];
#pragma unroll
          for (int i = 0; i < NP; ++i) out[i] = __ffma2_rn(__fmul2_rn(X[j][i], r2), sc[i], sh[i]);
          Vec<T, VEC> o;
          pack2<T, VEC>(out, o);
          o.store(out_p);
        }
        out_p += H;
      }
    }
    if (++stage == a.stages) {
      stage = 0;
      parity ^= 1u;
    }
    yp += group_elems;
    if constexpr (RES) xn += group_elems;
    if (inv_p != nullptr) {
      inv_p += RPI;
      if constexpr (!RMS) mean_p += RPI;
    }
    return true;
  };

  const int n_full = n / RPI;
  for (int g = 0; g < n_full; ++g) {
    if (!group(std::true_type{}, RPI)) {
      drain_after_abort();
      return;
    }
  }
  if (n_full < n_groups) {
    if (!group(std::false_type{}, n - n_full * RPI)) {
      drain_after_abort();
      return;
    }
  }
}

// The backward (dx, column sums, or both in one pass) for the launch plan that nearly every training shape gets:
// every chunk lies inside one sample (`chunks_per_sample` > 0). Same pipeline, same arithmetic in the same order and
// the same workspace slots as norm_bwd_tma - results are bit-identical - but the walk is flat: the chunk
// is `n` rows of one sample, so there is no sample cursor, the modulation vector and the column accumulators are
// set up once, row and byte positions are 32-bit offsets from bases computed once, and the groups of RPI rows
// run through a body without row predicates; only a ragged last group takes the predicated body. At H = 1152 that
// is about a sixth fewer instructions per row, and at this size time follows the instruction count.
template <typename T, int VEC, int RPI, int MAXR, bool RMS, bool DX = true, bool DP = true>
__global__ void __maxnreg__(MAXR) norm_bwd_tma_flat(const NormArgs a) {
  constexpr int NP = VEC / 2;
  constexpr int Q = RMS ? 1 : 2;  // row sums needed for dx: [sum dxhat,] sum dxhat*xhat
  extern __shared__ __align__(128) unsigned char dsm[];
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm);
  unsigned char* buf = dsm + kBarrierBytes;
  __shared__ __align__(16) float red[2][Q * RPI * 32];
  __shared__ __align__(16) float zero16[4];
  __shared__ int s_abort;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  if (tid < 4) zero16[tid] = 0.f;
  if (tid == 0) s_abort = 0;

  const int H = a.hidden;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const uint32_t stage_total = 2 * RPI * row_bytes;  // x rows then dy rows
  const bool active = tid < H / VEC;
  const int col = active ? tid * VEC : 0;
  const uint32_t src_stride = active ? row_bytes : 0u;
  const uint32_t dy_off = active ? RPI * row_bytes : 0u;
  const float inv_h = 1.f / static_cast<float>(H);

  // this CTA's chunk: rows [r0, r0 + n) of sample bi of the shard (whole samples, cut evenly)
  const int k = a.chunks_per_sample, seq = static_cast<int>(a.seq_len);
  const int bi = static_cast<int>(blockIdx.x) / k, cj = static_cast<int>(blockIdx.x) - bi * k;
  const int cbase = seq / k, crem = seq - cbase * k;
  const long long r0 = static_cast<long long>(bi) * seq + cj * cbase + (cj < crem ? cj : crem);
  const int n = cbase + (cj < crem ? 1 : 0);
  const int n_groups = (n + RPI - 1) / RPI;
  const long long b = a.b_first + bi;

  if (tid == 0) {
    for (int s = 0; s < a.stages; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  griddep_wait();  // nothing above reads global memory; everything below may

  // thread 0 keeps `stages` groups in flight: group g of the chunk goes to stage g % stages
  const T* xg = static_cast<const T*>(a.x) + r0 * H;
  const T* gg = static_cast<const T*>(a.dy) + r0 * H;
  int pg = 0;  // next group to request (thread 0 only)
  auto request = [&](int g, int s) {
    const int rows = n - g * RPI < RPI ? n - g * RPI : RPI;
    const uint32_t bytes = static_cast<uint32_t>(rows) * row_bytes;
    unsigned char* dst = buf + static_cast<uint32_t>(s) * stage_total;
    const size_t off = static_cast<size_t>(g) * RPI * H;
    mbar_expect_tx(&full[s], 2 * bytes);
    bulk_load_1d(dst, xg + off, bytes, &full[s]);
    bulk_load_1d(dst + RPI * row_bytes, gg + off, bytes, &full[s]);
  };
  if (tid == 0) {
    for (int s = 0; s < a.stages && pg < n_groups; ++s, ++pg) {
      // test switch: CTA 0 never sends its first group, so the wait on stage 0 expires with nothing in flight
      if (!(a.withhold_first_copy && blockIdx.x == 0 && s == 0)) request(pg, s);
    }
  }

  [[maybe_unused]] float2 sc1[NP], acc_s[NP], acc_h[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) acc_s[i] = acc_h[i] = make_float2(0.f, 0.f);
  if constexpr (DX) {
    Vec<T, VEC> vs;
    vs.load(static_cast<const T*>(a.scale) + b * H + col);
    unpack2<T, VEC>(vs, sc1);
#pragma unroll
    for (int i = 0; i < NP; ++i) sc1[i] = __fadd2_rn(sc1[i], make_float2(1.f, 1.f));
  }
  const float* inv_p = a.invstd + r0;
  const float* mean_p = RMS ? nullptr : a.mean + r0;
  [[maybe_unused]] T* dp = DX ? static_cast<T*>(a.dx) + r0 * H + col : nullptr;
  const size_t group_elems = static_cast<size_t>(RPI) * H;
  int stage = 0, phase = 0;
  uint32_t parity = 0;

  // one group of rows; FULL: all RPI rows exist (no row predicates). Returns false when the CTA must leave.
  auto group = [&](auto full_tag, int nrows) -> bool {
    constexpr bool FULL = decltype(full_tag)::value;
    float rstd[RPI], nmean[RPI];
#pragma unroll
    for (int j = 0; j < RPI; ++j) {
      const int jj = FULL || j < nrows ? j : nrows - 1;  // clamped inside the group
      rstd[j] = __ldg(inv_p + jj);
      if constexpr (!RMS) nmean[j] = -__ldg(mean_p + jj);
      else nmean[j] = 0.f;
    }
    if (!mbar_wait_1s(&full[stage], parity, a.err, 2, a.wait_limit_ns)) s_abort = 1;  // seen by all after the next barrier
    const unsigned char* src =
        active ? buf + static_cast<uint32_t>(stage) * stage_total + col * sizeof(T) : reinterpret_cast<const unsigned char*>(zero16);
    float2 X[RPI][NP], G[RPI][NP];
#pragma unroll
    for (int j = 0; j < RPI; ++j) {
      Vec<T, VEC> px, pgv;
      *reinterpret_cast<uint4*>(px.v) = *reinterpret_cast<const uint4*>(src + j * src_stride);
      *reinterpret_cast<uint4*>(pgv.v) = *reinterpret_cast<const uint4*>(src + dy_off + j * src_stride);
      unpack2<T, VEC>(px, X[j]);
      unpack2<T, VEC>(pgv, G[j]);
    }
    if constexpr (!FULL) {  // rows past the group's end hold stale data: keep them out of the column sums
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        if (j >= nrows) {
#pragma unroll
          for (int i = 0; i < NP; ++i) {
            G[j][i] = make_float2(0.f, 0.f);
            X[j][i] = make_float2(0.f, 0.f);
          }
        }
      }
    }
    float p[Q][RPI];
#pragma unroll
    for (int j = 0; j < RPI; ++j) {
      const float2 r2 = make_float2(rstd[j], rstd[j]), m2 = make_float2(nmean[j], nmean[j]);
      float2 p0 = make_float2(0.f, 0.f), p1 = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        if constexpr (!RMS) X[j][i] = __fadd2_rn(X[j][i], m2);
        X[j][i] = __fmul2_rn(X[j][i], r2);  // xhat in place
        if constexpr (DP) {
          acc_h[i] = __fadd2_rn(acc_h[i], G[j][i]);
          acc_s[i] = __ffma2_rn(G[j][i], X[j][i], acc_s[i]);
        }
        if constexpr (DX) {
          G[j][i] = __fmul2_rn(G[j][i], sc1[i]);  // dxhat in place
          if constexpr (!RMS) p0 = __fadd2_rn(p0, G[j][i]);
          p1 = __ffma2_rn(G[j][i], X[j][i], p1);
        }
      }
      if constexpr (DX) {
        if constexpr (!RMS) p[0][j] = p0.x + p0.y;
        p[Q - 1][j] = p1.x + p1.y;
      }
    }
    if constexpr (DX) {
      float mine[Q];
      cta_sum_rows_post<Q, RPI>(p, mine, red[phase], lane, warp, warps,
                                [&](int, float t) { return -t * inv_h; });  // broadcast -mean_h(.)
      phase ^= 1;
    } else {
      __syncthreads();  // every thread has read the stage
    }
    if (*static_cast<volatile int*>(&s_abort)) return false;
    if (tid == 0 && pg < n_groups) {  // every thread has read the stage: refill it
      fence_proxy_async_smem();
      request(pg, stage);
      ++pg;
    }
    if (++stage == a.stages) {
      stage = 0;
      parity ^= 1u;
    }
    if (DX && active) {
      T* out_p = dp;
#pragma unroll
      for (int j = 0; j < RPI; ++j) {
        if (FULL || j < nrows) {
          const float2 c2v = make_float2(p[Q - 1][j], p[Q - 1][j]), r2 = make_float2(rstd[j], rstd[j]);
          float2 out[NP];
#pragma unroll
          for (int i = 0; i < NP; ++i) {
            float2 t = G[j][i];
            if constexpr (!RMS) t = __fadd2_rn(t, make_float2(p[0][j], p[0][j]));
            t = __ffma2_rn(X[j][i], c2v, t);
            out[i] = __fmul2_rn(t, r2);
          }
          Vec<T, VEC> o;
          pack2<T, VEC>(out, o);
          o.store(out_p);
        }
        out_p += H;
      }
    }
    inv_p += RPI;
    if constexpr (!RMS) mean_p += RPI;
    if constexpr (DX) dp += group_elems;
    return true;
  };

  const int n_full = n / RPI;
  for (int g = 0; g < n_full; ++g) {
    // The kernels that depend on this launch (stage 2, then whatever follows) are released when the last full group
    // begins, not at entry: released at entry they sit in the CTA slots that free up first while the launch after
    // them cannot start - measured 16.2 us per backward + stage 2 in a loop of them against 15.0 us this way, and a
    // step 0.6 - 0.9 us shorter (AdaLN / AdaRMSNorm at the DiT-XL/2 shape).
    if (g == n_full - 1) griddep_launch_dependents();
    if (!group(std::true_type{}, RPI)) {
      drain_after_abort();
      return;
    }
  }
  if (n_full < n_groups) {
    if (!group(std::false_type{}, n - n_full * RPI)) {
      drain_after_abort();
      return;
    }
  }

  // stage 1 of the dparam reduction: this chunk's column sums go to its own workspace slot
  if (DP && active) {
    constexpr int NF4 = VEC / 4;  // float4 chunks per thread (VEC is 4 or 8)
    float* part = a.ws_part + (static_cast<long long>(blockIdx.x) + bi) * 2 * H + col;
#pragma unroll
    for (int kk = 0; kk < NF4; ++kk) {
      reinterpret_cast<float4*>(part)[kk] = make_float4(acc_s[2 * kk].x, acc_s[2 * kk].y, acc_s[2 * kk + 1].x, acc_s[2 * kk + 1].y);
      reinterpret_cast<float4*>(part + H)[kk] = make_float4(acc_h[2 * kk].x, acc_h[2 * kk].y, acc_h[2 * kk + 1].x, acc_h[2 * kk + 1].y);
    }
  }
}

template <typename T, int VEC, int RPI, int MAXRF, int MAXRB>
static const void* pick_tma_flat_fwd(bool rms, bool res) {
  if (res)
    return rms ? (const void*)norm_fwd_tma_flat<T, VEC, RPI, MAXRB, true, true> : (const void*)norm_fwd_tma_flat<T, VEC, RPI, MAXRB, false, true>;
  return rms ? (const void*)norm_fwd_tma_flat<T, VEC, RPI, MAXRF, true> : (const void*)norm_fwd_tma_flat<T, VEC, RPI, MAXRF, false>;
}

template <typename T, int VEC, int RPI, int MAXRB>
static const void* pick_tma_flat_bwd(int mode, bool rms) {
  switch (mode) {
    case kBwdDx:
      return rms ? (const void*)norm_bwd_tma_flat<T, VEC, RPI, MAXRB, true, true, false>
                 : (const void*)norm_bwd_tma_flat<T, VEC, RPI, MAXRB, false, true, false>;
    case kBwdDparam:
      return rms ? (const void*)norm_bwd_tma_flat<T, VEC, RPI, MAXRB, true, false, true>
                 : (const void*)norm_bwd_tma_flat<T, VEC, RPI, MAXRB, false, false, true>;
    default:
      return rms ? (const void*)norm_bwd_tma_flat<T, VEC, RPI, MAXRB, true> : (const void*)norm_bwd_tma_flat<T, VEC, RPI, MAXRB, false>;
  }
}

template <typename T, int VEC, int RPI, int MAXRF, int MAXRB>
static const void* pick_tma(int mode, bool rms, bool res = false) {
  if (mode == kFwd && res)
    return rms ? (const void*)norm_fwd_tma<T, VEC, RPI, MAXRB, true, true> : (const void*)norm_fwd_tma<T, VEC, RPI, MAXRB, false, true>;
  switch (mode) {
    case kFwd:
      return rms ? (const void*)norm_fwd_tma<T, VEC, RPI, MAXRF, true> : (const void*)norm_fwd_tma<T, VEC, RPI, MAXRF, false>;
    case kBwdDx:
      return rms ? (const void*)norm_bwd_tma<T, VEC, RPI, MAXRB, true, true, false>
                 : (const void*)norm_bwd_tma<T, VEC, RPI, MAXRB, false, true, false>;
    case kBwdDparam:
      return rms ? (const void*)norm_bwd_tma<T, VEC, RPI, MAXRB, true, false, true>
                 : (const void*)norm_bwd_tma<T, VEC, RPI, MAXRB, false, false, true>;
    default:
      return rms ? (const void*)norm_bwd_tma<T, VEC, RPI, MAXRB, true, true, true>
                 : (const void*)norm_bwd_tma<T, VEC, RPI, MAXRB, false, true, true>;
  }
}

}  // namespace nd
