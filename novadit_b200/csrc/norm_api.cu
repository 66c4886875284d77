// C entry points of the AdaLN / AdaRMSNorm operators: argument checks, tile
// plan, workspace layout, dispatch on element type.
#include <atomic>

#include "norm_impl.cuh"

namespace nd {

int launch_norm_f16(const NormArgs& a, cudaStream_t st);
int launch_norm_bf16(const NormArgs& a, cudaStream_t st);
int launch_norm_f32(const NormArgs& a, cudaStream_t st);

static std::atomic<int> g_tile_rows_override{0};
int tile_rows_override() { return g_tile_rows_override.load(std::memory_order_relaxed); }

TilePlan plan_tiles(long long rows, long long row_start, long long seq_len, int tile_rows) {
  TilePlan p{};
  if (rows <= 0 || seq_len <= 0) return p;
  p.b_first = row_start / seq_len;
  const long long b_last = (row_start + rows - 1) / seq_len;
  p.n_samples = b_last - p.b_first + 1;
  p.tile_rows = tile_rows < 1 ? 1 : tile_rows;
  p.tiles_per_sample = static_cast<int>((seq_len + p.tile_rows - 1) / p.tile_rows);
  p.n_items = p.n_samples * p.tiles_per_sample;
  return p;
}

// Workspace: [counters: n_samples x u32, padded to 256 B][partials: items x 2 x H fp32], sized for
// the finest tiling the launcher may choose (8-row tiles, or the override if smaller).
static size_t counter_bytes(const TilePlan& p) {
  return (static_cast<size_t>(p.n_samples) * sizeof(unsigned int) + 255) / 256 * 256;
}

static TilePlan finest_plan(long long rows, long long row_start, long long seq_len) {
  int tr = 8;
  const int forced = tile_rows_override();
  if (forced > 0 && forced < tr) tr = forced;
  return plan_tiles(rows, row_start, seq_len, tr);
}

static int check_shape(int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden) {
  if (rows < 0 || row_start < 0 || seq_len <= 0 || hidden <= 0) return ND_ERR_BAD_ARG;
  if (seq_len > INT32_MAX || hidden > INT32_MAX) return ND_ERR_UNSUPPORTED;
  return ND_OK;
}

static int dispatch(int dtype, const NormArgs& a, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case ND_F16: return launch_norm_f16(a, st);
    case ND_BF16: return launch_norm_bf16(a, st);
    case ND_F32: return launch_norm_f32(a, st);
    default: return ND_ERR_UNSUPPORTED;
  }
}

static int norm_fwd(bool rms, int dtype, const void* x, const void* scale, const void* shift,
                    void* y, float* mean, float* invstd, int64_t rows, int64_t row_start,
                    int64_t seq_len, int64_t hidden, float eps, void* stream) {
  if (int s = check_shape(rows, row_start, seq_len, hidden)) return s;
  if (rows == 0) return ND_OK;
  if (!x || !scale || !shift || !y) return ND_ERR_BAD_ARG;
  if (!rms && ((mean == nullptr) != (invstd == nullptr))) return ND_ERR_BAD_ARG;
  NormArgs a{};
  a.x = x; a.scale = scale; a.shift = shift; a.y = y;
  a.mean = rms ? nullptr : mean;
  a.invstd = invstd;
  a.rows = rows; a.row_start = row_start;
  a.seq_len = static_cast<int>(seq_len); a.hidden = static_cast<int>(hidden);
  a.eps = eps; a.mode = kFwd; a.rms = rms;
  return dispatch(dtype, a, stream);
}

static int norm_bwd(bool rms, int mode, int dtype, const void* dy, const void* x,
                    const void* scale, const float* mean, const float* invstd, void* dx,
                    float* dscale, float* dshift, int64_t rows, int64_t row_start,
                    int64_t seq_len, int64_t hidden, void* ws, size_t ws_bytes, void* stream) {
  if (int s = check_shape(rows, row_start, seq_len, hidden)) return s;
  if (rows == 0) return ND_OK;
  const bool want_dx = mode != kBwdDparam, want_dp = mode != kBwdDx;
  if (!dy || !x || !invstd || (!rms && !mean)) return ND_ERR_BAD_ARG;
  if (want_dx && (!scale || !dx)) return ND_ERR_BAD_ARG;
  if (want_dp && (!dscale || !dshift)) return ND_ERR_BAD_ARG;
  NormArgs a{};
  a.dy = dy; a.x = x; a.scale = scale; a.dx = dx;
  a.mean = const_cast<float*>(rms ? nullptr : mean);
  a.invstd = const_cast<float*>(invstd);
  a.dscale = dscale; a.dshift = dshift;
  a.rows = rows; a.row_start = row_start;
  a.seq_len = static_cast<int>(seq_len); a.hidden = static_cast<int>(hidden);
  a.mode = mode; a.rms = rms;
  if (want_dp) {
    const size_t need = nd_norm_dparam_ws_bytes(rows, row_start, seq_len, hidden);
    if (need > 0) {
      if (!ws || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u)) return ND_ERR_WORKSPACE;
      const TilePlan p = finest_plan(rows, row_start, seq_len);
      a.ws_cnt = static_cast<unsigned int*>(ws);
      a.ws_part = reinterpret_cast<float*>(static_cast<char*>(ws) + counter_bytes(p));
    }
  }
  return dispatch(dtype, a, stream);
}

}  // namespace nd

using namespace nd;

extern "C" {

// Tuning hook used by the benchmark sweeps: force the row-tile height of the
// norm kernels (0 restores the built-in choice). Process-wide.
void nd_tune_norm_tile_rows(int tile_rows) { g_tile_rows_override.store(tile_rows < 0 ? 0 : tile_rows); }

size_t nd_norm_dparam_ws_counter_bytes(int64_t rows, int64_t row_start, int64_t seq_len,
                                       int64_t hidden) {
  if (check_shape(rows, row_start, seq_len, hidden) != ND_OK || rows == 0) return 0;
  return counter_bytes(finest_plan(rows, row_start, seq_len));
}

size_t nd_norm_dparam_ws_bytes(int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden) {
  if (check_shape(rows, row_start, seq_len, hidden) != ND_OK || rows == 0) return 0;
  const TilePlan p = finest_plan(rows, row_start, seq_len);
  if (p.tiles_per_sample <= 1) return 0;
  return counter_bytes(p) + static_cast<size_t>(p.n_items) * 2 * static_cast<size_t>(hidden) * sizeof(float);
}

int nd_norm_dparam_ws_init(void* ws, size_t ws_bytes, int64_t rows, int64_t row_start,
                           int64_t seq_len, int64_t hidden, void* stream) {
  const size_t need = nd_norm_dparam_ws_bytes(rows, row_start, seq_len, hidden);
  if (need == 0) return ND_OK;
  if (!ws || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u)) return ND_ERR_WORKSPACE;
  const size_t cb = nd_norm_dparam_ws_counter_bytes(rows, row_start, seq_len, hidden);
  cudaError_t e = cudaMemsetAsync(ws, 0, cb, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}

int nd_adaln_fwd(int dtype, const void* x, const void* scale, const void* shift, void* y,
                 float* mean, float* invstd, int64_t rows, int64_t row_start, int64_t seq_len,
                 int64_t hidden, float eps, void* stream) {
  return norm_fwd(false, dtype, x, scale, shift, y, mean, invstd, rows, row_start, seq_len, hidden,
                  eps, stream);
}

int nd_adaln_bwd_dx(int dtype, const void* dy, const void* x, const void* scale,
                    const float* mean, const float* invstd, void* dx, int64_t rows,
                    int64_t row_start, int64_t seq_len, int64_t hidden, void* stream) {
  return norm_bwd(false, kBwdDx, dtype, dy, x, scale, mean, invstd, dx, nullptr, nullptr, rows,
                  row_start, seq_len, hidden, nullptr, 0, stream);
}

int nd_adaln_bwd_dparam(int dtype, const void* dy, const void* x, const float* mean,
                        const float* invstd, float* dscale, float* dshift, int64_t rows,
                        int64_t row_start, int64_t seq_len, int64_t hidden, void* ws,
                        size_t ws_bytes, void* stream) {
  return norm_bwd(false, kBwdDparam, dtype, dy, x, nullptr, mean, invstd, nullptr, dscale, dshift,
                  rows, row_start, seq_len, hidden, ws, ws_bytes, stream);
}

int nd_adaln_bwd(int dtype, const void* dy, const void* x, const void* scale, const float* mean,
                 const float* invstd, void* dx, float* dscale, float* dshift, int64_t rows,
                 int64_t row_start, int64_t seq_len, int64_t hidden, void* ws, size_t ws_bytes,
                 void* stream) {
  return norm_bwd(false, kBwdFused, dtype, dy, x, scale, mean, invstd, dx, dscale, dshift, rows,
                  row_start, seq_len, hidden, ws, ws_bytes, stream);
}

int nd_adarms_fwd(int dtype, const void* x, const void* scale, const void* shift, void* y,
                  float* inv_rms, int64_t rows, int64_t row_start, int64_t seq_len,
                  int64_t hidden, float eps, void* stream) {
  return norm_fwd(true, dtype, x, scale, shift, y, nullptr, inv_rms, rows, row_start, seq_len,
                  hidden, eps, stream);
}

int nd_adarms_bwd_dx(int dtype, const void* dy, const void* x, const void* scale,
                     const float* inv_rms, void* dx, int64_t rows, int64_t row_start,
                     int64_t seq_len, int64_t hidden, void* stream) {
  return norm_bwd(true, kBwdDx, dtype, dy, x, scale, nullptr, inv_rms, dx, nullptr, nullptr, rows,
                  row_start, seq_len, hidden, nullptr, 0, stream);
}

int nd_adarms_bwd_dparam(int dtype, const void* dy, const void* x, const float* inv_rms,
                         float* dscale, float* dshift, int64_t rows, int64_t row_start,
                         int64_t seq_len, int64_t hidden, void* ws, size_t ws_bytes,
                         void* stream) {
  return norm_bwd(true, kBwdDparam, dtype, dy, x, nullptr, nullptr, inv_rms, nullptr, dscale,
                  dshift, rows, row_start, seq_len, hidden, ws, ws_bytes, stream);
}

int nd_adarms_bwd(int dtype, const void* dy, const void* x, const void* scale,
                  const float* inv_rms, void* dx, float* dscale, float* dshift, int64_t rows,
                  int64_t row_start, int64_t seq_len, int64_t hidden, void* ws, size_t ws_bytes,
                  void* stream) {
  return norm_bwd(true, kBwdFused, dtype, dy, x, scale, nullptr, inv_rms, dx, dscale, dshift, rows,
                  row_start, seq_len, hidden, ws, ws_bytes, stream);
}

}  // extern "C"
