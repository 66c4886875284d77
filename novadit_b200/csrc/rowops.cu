// The two row operators the reference specifies but never implemented (sm_100a):
//   out-residual  y = x + residual (+ bias[h])            novadit/ops/residual.py:8-25, stub csrc/ops/residual_kernel.cu
//   QKV pack      [rows, 3H] -> q, k, v [rows, H] (+ back) novadit/ops/qkv_pack.py:9-44, stub csrc/ops/qkv_pack_kernel.cu
//   gated residual y = x + gate[b] * branch and its backward (dbranch, dgate): the adaLN-Zero residual of DiT blocks
// Pure streaming work, laid out like the gate-act kernels: one CTA per row, thread t handles 16-byte vectors
// t, t + NT, ... of the row, fp32 math for the sum, one rounding on store. Misaligned or odd-width rows take
// the same kernels with one element per "vector".
#include "common.cuh"

namespace nd {

struct ResidualArgs {
  const void* x;
  const void* residual;
  const void* bias;  // [hidden] or null
  void* y;
  long long rows;
  int hidden;
};

template <typename T, int VEC>
__global__ void __launch_bounds__(256) out_residual_kernel(const ResidualArgs a) {
  const int nvec = a.hidden / VEC;
  const T* __restrict__ bias = static_cast<const T*>(a.bias);
  for (long long row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const T* __restrict__ x = static_cast<const T*>(a.x) + row * a.hidden;
    const T* __restrict__ r = static_cast<const T*>(a.residual) + row * a.hidden;
    T* __restrict__ y = static_cast<T*>(a.y) + row * a.hidden;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      Vec<T, VEC> vx, vr, vb;
      vx.load_stream(x + v * VEC);
      vr.load_stream(r + v * VEC);
      float fx[VEC], fr[VEC], fb[VEC];
      vx.unpack(fx);
      vr.unpack(fr);
      if (bias != nullptr) {
        vb.load(bias + v * VEC);
        vb.unpack(fb);
      } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) fb[k] = 0.f;
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) fx[k] = (fx[k] + fr[k]) + fb[k];
      Vec<T, VEC> o;
      o.pack(fx);
      o.store(y + v * VEC);
    }
  }
}

struct QkvArgs {
  void* qkv;      // [rows, 3H]
  void* part[3];  // q, k, v: [rows, H] each
  long long rows;
  int hidden;
};

// PACK: qkv -> q, k, v; otherwise q, k, v -> qkv (the backward of the pack)
template <typename T, int VEC, bool PACK>
__global__ void __launch_bounds__(256) qkv_pack_kernel(const QkvArgs a) {
  const int nvec = a.hidden / VEC;
  for (long long row = blockIdx.x; row < a.rows; row += gridDim.x) {
    T* wide = static_cast<T*>(a.qkv) + row * 3LL * a.hidden;
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      T* narrow = static_cast<T*>(a.part[p]) + row * a.hidden;
      T* w = wide + static_cast<long long>(p) * a.hidden;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        Vec<T, VEC> t;
        if (PACK) {
          t.load_stream(w + v * VEC);
          t.store(narrow + v * VEC);
        } else {
          t.load_stream(narrow + v * VEC);
          t.store(w + v * VEC);
        }
      }
    }
  }
}

// Gated residual of adaLN-Zero blocks: y = x + gate[b, :] * branch over rows of sample b (forward), and
// dbranch = gate * dy with the per-sample column sums of dy * branch for dgate (backward). A CTA takes TR
// consecutive rows of one sample; thread t owns column vectors t, t + NT, ...; the backward keeps its column sums in
// registers and writes one fp32 partial row per (sample, tile) - summed over tiles by the caller in a fixed order.
struct GatedArgs {
  const void* a;     // forward: x; backward: dy
  const void* b;     // branch
  const void* gate;  // [batch, hidden]
  void* out;         // forward: y; backward: dbranch
  float* part;       // backward: [batch_in_shard * tiles_per_sample, hidden] fp32
  const void* add;   // backward, nullable: a second gradient of the same tensor, added to dy first
  void* sum_out;     // backward with `add`: dy + add, rounded once (what flows on along the residual stream)
  long long rows, row_start;
  int seq_len, hidden, tile_rows, tiles_per_sample;
  long long b_first;
};

template <typename T, int VEC, bool BWD>
__global__ void __launch_bounds__(256) gated_residual_kernel(const GatedArgs g) {
  const int nvec = g.hidden / VEC;
  const long long item = blockIdx.x;
  const long long bi = item / g.tiles_per_sample;
  const int tile = static_cast<int>(item - bi * g.tiles_per_sample);
  const long long b = g.b_first + bi;
  // rows of this tile, global -> clipped to the shard -> local
  long long g0 = b * g.seq_len + static_cast<long long>(tile) * g.tile_rows;
  long long g1 = g0 + g.tile_rows;
  const long long gend = (b + 1) * g.seq_len;
  if (g1 > gend) g1 = gend;
  const long long lo = g.row_start, hi = g.row_start + g.rows;
  const long long l0 = (g0 > lo ? g0 : lo) - lo, l1 = (g1 < hi ? g1 : hi) - lo;
  const T* __restrict__ pa = static_cast<const T*>(g.a);
  const T* __restrict__ pb = static_cast<const T*>(g.b);
  T* __restrict__ po = static_cast<T*>(g.out);
  [[maybe_unused]] const T* __restrict__ padd = static_cast<const T*>(g.add);
  [[maybe_unused]] T* __restrict__ psum = static_cast<T*>(g.sum_out);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    Vec<T, VEC> vg;
    vg.load(static_cast<const T*>(g.gate) + b * g.hidden + v * VEC);
    float fg[VEC], acc[VEC];
    vg.unpack(fg);
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
    for (long long r = l0; r < l1; r += 4) {
      Vec<T, VEC> va[4], vb[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        va[j].zero();
        vb[j].zero();
        if (r + j < l1) {
          va[j].load_stream(pa + (r + j) * g.hidden + v * VEC);
          vb[j].load_stream(pb + (r + j) * g.hidden + v * VEC);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (r + j < l1) {
          float fa[VEC], fb[VEC], fo[VEC];
          va[j].unpack(fa);
          vb[j].unpack(fb);
          if constexpr (BWD) {
            if (padd != nullptr) {  // dy + add, rounded to T as the separate addition would: the rest uses that value
              Vec<T, VEC> vd;
              vd.load_stream(padd + (r + j) * g.hidden + v * VEC);
              float fd[VEC];
              vd.unpack(fd);
#pragma unroll
              for (int k = 0; k < VEC; ++k) fa[k] += fd[k];
              vd.pack(fa);
              vd.store(psum + (r + j) * g.hidden + v * VEC);
              vd.unpack(fa);
            }
          }
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            if constexpr (BWD) {
              fo[k] = fg[k] * fa[k];            // dbranch = gate * dy
              acc[k] = fmaf(fa[k], fb[k], acc[k]);  // dgate += dy * branch
            } else {
              fo[k] = fmaf(fg[k], fb[k], fa[k]);    // y = x + gate * branch
            }
          }
          Vec<T, VEC> o;
          o.pack(fo);
          o.store(po + (r + j) * g.hidden + v * VEC);
        }
      }
    }
    if constexpr (BWD) {
      float* dst = g.part + item * g.hidden + v * VEC;
#pragma unroll
      for (int k = 0; k < VEC; ++k) dst[k] = acc[k];
    }
  }
}

static int threads_for(int nvec) {
  const int passes = (nvec + 255) / 256;
  int nt = ((nvec + passes - 1) / passes + 31) / 32 * 32;
  return nt < 32 ? 32 : nt;
}

static int launch(const void* fn, void* args, long long rows, int nt, cudaStream_t st) {
  long long grid = rows < 0x7FFFFFFFLL ? rows : 0x7FFFFFFFLL;  // the kernels stride over rows
  if (grid < 1) return ND_OK;
  void* params[] = {args};
  cudaError_t e = cudaLaunchKernel(fn, dim3(static_cast<unsigned>(grid)), dim3(nt), params, 0, st);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}

template <typename T>
static int launch_residual(ResidualArgs a, cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(T);
  const bool vec_ok = a.hidden % VMAX == 0 && aligned16(a.x) && aligned16(a.residual) && aligned16(a.y) &&
                      aligned16(a.bias);
  if (vec_ok) return launch(reinterpret_cast<const void*>(out_residual_kernel<T, VMAX>), &a, a.rows, threads_for(a.hidden / VMAX), st);
  return launch(reinterpret_cast<const void*>(out_residual_kernel<T, 1>), &a, a.rows, threads_for(a.hidden), st);
}

template <typename T>
static int launch_qkv(QkvArgs a, bool pack, cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(T);
  const bool vec_ok = a.hidden % VMAX == 0 && aligned16(a.qkv) && aligned16(a.part[0]) && aligned16(a.part[1]) &&
                      aligned16(a.part[2]);
  const void* fn;
  if (vec_ok) fn = pack ? (const void*)qkv_pack_kernel<T, VMAX, true> : (const void*)qkv_pack_kernel<T, VMAX, false>;
  else fn = pack ? (const void*)qkv_pack_kernel<T, 1, true> : (const void*)qkv_pack_kernel<T, 1, false>;
  return launch(fn, &a, a.rows, threads_for(vec_ok ? a.hidden / VMAX : a.hidden), st);
}

static int qkv_entry(int dtype, bool pack, void* qkv, void* q, void* k, void* v, int64_t rows, int64_t hidden,
                     void* stream) {
  if (rows < 0 || hidden <= 0) return ND_ERR_BAD_ARG;
  if (hidden > INT32_MAX / 3) return ND_ERR_UNSUPPORTED;
  if (rows == 0) return ND_OK;
  if (!qkv || !q || !k || !v) return ND_ERR_BAD_ARG;
  QkvArgs a{qkv, {q, k, v}, rows, static_cast<int>(hidden)};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case ND_F16: return launch_qkv<__half>(a, pack, st);
    case ND_BF16: return launch_qkv<__nv_bfloat16>(a, pack, st);
    case ND_F32: return launch_qkv<float>(a, pack, st);
    default: return ND_ERR_UNSUPPORTED;
  }
}

static int gated_entry(int dtype, bool bwd, const void* a, const void* b, const void* gate, void* out, float* part,
                       int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden, int64_t tile_rows,
                       void* stream, const void* add = nullptr, void* sum_out = nullptr) {
  if (rows < 0 || row_start < 0 || seq_len <= 0 || hidden <= 0 || tile_rows <= 0) return ND_ERR_BAD_ARG;
  if (hidden > INT32_MAX || seq_len > INT32_MAX || tile_rows > INT32_MAX) return ND_ERR_UNSUPPORTED;
  if (rows == 0) return ND_OK;
  if (!a || !b || !gate || !out || (bwd && !part) || ((add != nullptr) != (sum_out != nullptr))) return ND_ERR_BAD_ARG;
  GatedArgs g{};
  g.add = add; g.sum_out = sum_out;
  g.a = a; g.b = b; g.gate = gate; g.out = out; g.part = part;
  g.rows = rows; g.row_start = row_start;
  g.seq_len = static_cast<int>(seq_len); g.hidden = static_cast<int>(hidden);
  g.tile_rows = static_cast<int>(tile_rows);
  g.tiles_per_sample = static_cast<int>((seq_len + tile_rows - 1) / tile_rows);
  g.b_first = row_start / seq_len;
  const long long n_samples = (row_start + rows - 1) / seq_len - g.b_first + 1;
  const long long items = n_samples * g.tiles_per_sample;
  if (items > 0x7FFFFFFFLL) return ND_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto go = [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VMAX = 16 / sizeof(T);
    const bool vec_ok = g.hidden % VMAX == 0 && aligned16(a) && aligned16(b) && aligned16(gate) && aligned16(out) &&
                        (!bwd || aligned16(part)) && aligned16(add) && aligned16(sum_out);
    const void* fn;
    if (vec_ok) fn = bwd ? (const void*)gated_residual_kernel<T, VMAX, true> : (const void*)gated_residual_kernel<T, VMAX, false>;
    else fn = bwd ? (const void*)gated_residual_kernel<T, 1, true> : (const void*)gated_residual_kernel<T, 1, false>;
    void* params[] = {&g};
    cudaError_t e = cudaLaunchKernel(fn, dim3(static_cast<unsigned>(items)), dim3(threads_for(vec_ok ? g.hidden / VMAX : g.hidden)),
                                     params, 0, st);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      (void)cudaGetLastError();
      return ND_ERR_LAUNCH;
    }
    return ND_OK;
  };
  switch (dtype) {
    case ND_F16: return go(__half{});
    case ND_BF16: return go(__nv_bfloat16{});
    case ND_F32: return go(float{});
    default: return ND_ERR_UNSUPPORTED;
  }
}

}  // namespace nd

extern "C" {

int nd_gated_residual_fwd(int dtype, const void* x, const void* branch, const void* gate, void* y, int64_t rows,
                          int64_t row_start, int64_t seq_len, int64_t hidden, void* stream) {
  return nd::gated_entry(dtype, false, x, branch, gate, y, nullptr, rows, row_start, seq_len, hidden, 8, stream);
}

size_t nd_gated_residual_ws_bytes(int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden, int64_t tile_rows) {
  if (rows <= 0 || row_start < 0 || seq_len <= 0 || hidden <= 0 || tile_rows <= 0) return 0;
  const int64_t n_samples = (row_start + rows - 1) / seq_len - row_start / seq_len + 1;
  return static_cast<size_t>(n_samples) * static_cast<size_t>((seq_len + tile_rows - 1) / tile_rows) *
         static_cast<size_t>(hidden) * sizeof(float);
}

int nd_gated_residual_bwd(int dtype, const void* dy, const void* branch, const void* gate, void* dbranch,
                          float* dgate_partials, int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden,
                          int64_t tile_rows, void* stream) {
  return nd::gated_entry(dtype, true, dy, branch, gate, dbranch, dgate_partials, rows, row_start, seq_len, hidden,
                         tile_rows, stream);
}


int nd_gated_residual_bwd_add(int dtype, const void* dy, const void* dres, const void* branch, const void* gate,
                              void* dsum, void* dbranch, float* dgate_partials, int64_t rows, int64_t row_start,
                              int64_t seq_len, int64_t hidden, int64_t tile_rows, void* stream) {
  if (!dres || !dsum) return ND_ERR_BAD_ARG;
  return nd::gated_entry(dtype, true, dy, branch, gate, dbranch, dgate_partials, rows, row_start, seq_len, hidden,
                         tile_rows, stream, dres, dsum);
}

int nd_out_residual_fwd(int dtype, const void* x, const void* residual, const void* bias, void* y, int64_t rows,
                        int64_t hidden, void* stream) {
  using namespace nd;
  if (rows < 0 || hidden <= 0) return ND_ERR_BAD_ARG;
  if (hidden > INT32_MAX) return ND_ERR_UNSUPPORTED;
  if (rows == 0) return ND_OK;
  if (!x || !residual || !y) return ND_ERR_BAD_ARG;
  ResidualArgs a{x, residual, bias, y, rows, static_cast<int>(hidden)};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case ND_F16: return launch_residual<__half>(a, st);
    case ND_BF16: return launch_residual<__nv_bfloat16>(a, st);
    case ND_F32: return launch_residual<float>(a, st);
    default: return ND_ERR_UNSUPPORTED;
  }
}

int nd_qkv_pack_fwd(int dtype, const void* qkv, void* q, void* k, void* v, int64_t rows, int64_t hidden,
                    void* stream) {
  return nd::qkv_entry(dtype, true, const_cast<void*>(qkv), q, k, v, rows, hidden, stream);
}

int nd_qkv_pack_bwd(int dtype, const void* dq, const void* dk, const void* dv, void* dqkv, int64_t rows,
                    int64_t hidden, void* stream) {
  return nd::qkv_entry(dtype, false, dqkv, const_cast<void*>(dq), const_cast<void*>(dk), const_cast<void*>(dv), rows,
                       hidden, stream);
}

}  // extern "C"

namespace nd {

// x + gate[b] * branch, or x + branch when there is no gate: the composed path of the norm forward with the
// residual in front, for rows the one-kernel version does not take
int gated_residual_fwd_any(int dtype, const void* x, const void* branch, const void* gate, void* y, int64_t rows,
                           int64_t row_start, int64_t seq_len, int64_t hidden, void* stream) {
  if (gate == nullptr) return nd_out_residual_fwd(dtype, x, branch, nullptr, y, rows, hidden, stream);
  return nd_gated_residual_fwd(dtype, x, branch, gate, y, rows, row_start, seq_len, hidden, stream);
}

}  // namespace nd
