// C entry points of the AdaLN / AdaRMSNorm operators: argument checks, tile
// plan, workspace layout, dispatch on element type.
#include <atomic>

#include "norm_launch.cuh"

namespace nd {

int launch_norm_f16(const NormArgs& a, cudaStream_t st);
int launch_norm_bf16(const NormArgs& a, cudaStream_t st);
int launch_norm_f32(const NormArgs& a, cudaStream_t st);

static std::atomic<int> g_tile_rows_override{0};
static std::atomic<int> g_norm_variant{0};
static std::atomic<int> g_norm_stages{0};
int norm_stages_override() { return g_norm_stages.load(std::memory_order_relaxed); }
static std::atomic<int> g_norm_cps{0};
int norm_chunks_per_sm() { return g_norm_cps.load(std::memory_order_relaxed); }
static std::atomic<int> g_norm_pdl{1};
int norm_pdl_enabled() { return g_norm_pdl.load(std::memory_order_relaxed); }
static std::atomic<unsigned long long> g_norm_wait_limit_ns{1000000000ull};
unsigned long long norm_wait_limit_ns() { return g_norm_wait_limit_ns.load(std::memory_order_relaxed); }
static std::atomic<int> g_norm_withhold{0};
int norm_withhold_first_copy() { return g_norm_withhold.load(std::memory_order_relaxed); }
int tile_rows_override() { return g_tile_rows_override.load(std::memory_order_relaxed); }
int norm_variant() { return g_norm_variant.load(std::memory_order_relaxed); }

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

// Workspace of the dparam reduction: fp32 partial column sums, one slot of [2][H] per (chunk, sample)
// segment of the bulk-copy kernels or per (sample, tile) item of the generic kernels, sized for the
// larger of the two upper bounds so that the caller need not know which kernel will run.
static size_t partial_slots(long long rows, long long row_start, long long seq_len) {
  int tr = 8;
  const int forced = tile_rows_override();
  if (forced > 0 && forced < tr) tr = forced;
  const TilePlan p = plan_tiles(rows, row_start, seq_len, tr);
  const long long chunk_slots = static_cast<long long>(sm_count()) * kMaxChunksPerSm + p.n_samples;
  return static_cast<size_t>(p.n_items > chunk_slots ? p.n_items : chunk_slots);
}

static int check_shape(int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden) {
  if (rows < 0 || row_start < 0 || seq_len <= 0 || hidden <= 0) return ND_ERR_BAD_ARG;
  if (seq_len > INT32_MAX || hidden > INT32_MAX) return ND_ERR_UNSUPPORTED;
  // every limit of the launches below is tested here, before the first kernel is enqueued: samples are a grid x
  // extent (2^31 - 1), the column blocks of the second dparam stage a grid y extent (65535)
  if (rows > 0 && (row_start + rows - 1) / seq_len - row_start / seq_len + 1 > INT32_MAX) return ND_ERR_UNSUPPORTED;
  if ((2 * hidden + 127) / 128 > 65535) return ND_ERR_UNSUPPORTED;
  return ND_OK;
}

// Stage 2 of the dparam reduction (any element type: the partials are fp32). Sample `b_first + blockIdx.x`
// (the grid's x extent has no practical limit: a 2-D input is one sample per row) owns the consecutive
// workspace slots [first, first + count); they are summed in index order.
//   chunk scheme (n_chunks > 0): slot = chunk + sample index, chunks = those that overlap the sample's rows;
//   item scheme  (n_chunks == 0): slot = sample index * tiles_per_sample + tile.
__global__ void __launch_bounds__(128) norm_dparam_stage2_kernel(const NormArgs a) {
  griddep_launch_dependents();
  griddep_wait();  // the partials come from the kernel launched just before
  const long long bi = blockIdx.x;
  const long long b = a.b_first + bi;
  const int H = a.hidden;
  long long first, count;
  if (a.n_chunks > 0 && a.chunks_per_sample > 0) {
    first = bi * a.chunks_per_sample + bi;  // slot = chunk + sample index, chunks [bi k, (bi + 1) k)
    count = a.chunks_per_sample;
  } else if (a.n_chunks > 0) {
    long long s0 = b * a.seq_len - a.row_start, s1 = s0 + a.seq_len;  // the sample's rows, local, clipped below
    if (s0 < 0) s0 = 0;
    if (s1 > a.rows) s1 = a.rows;
    if (s0 >= s1) return;
    // chunk holding row s: the first chunk_rem chunks have chunk_base + 1 rows, the others chunk_base
    const long long big = static_cast<long long>(a.chunk_rem) * (a.chunk_base + 1);
    auto chunk_of = [&](long long s) { return s < big ? s / (a.chunk_base + 1) : a.chunk_rem + (s - big) / a.chunk_base; };
    const long long c_lo = chunk_of(s0), c_hi = chunk_of(s1 - 1);
    first = c_lo + bi;
    count = c_hi - c_lo + 1;
  } else {
    first = bi * a.tiles_per_sample;
    count = a.tiles_per_sample;
  }
  const int colx = (blockIdx.y * blockDim.x + threadIdx.x);  // one column of [dscale | dshift] per thread
  if (colx >= 2 * H) return;
  const float* src = a.ws_part + first * 2 * H + colx;
  const long long stride = 2LL * H;
  float acc = 0.f;
  long long t = 0;
  constexpr int U = 16;  // independent loads in flight per round (a sample rarely has more partials than this)
  for (; t + U <= count; t += U) {  // summed in index order
    float v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = __ldcg(src + (t + u) * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) acc += v[u];
  }
  if (t < count) {
    float v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = t + u < count ? __ldcg(src + (t + u) * stride) : 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u) acc += v[u];  // adding +0 keeps the order and the value
  }
  float* dst = colx < H ? a.dscale + b * H + colx : a.dshift + b * H + (colx - H);
  *dst = acc;
}

int launch_dparam_stage2(const NormArgs& a, cudaStream_t st) {
  if (a.n_samples <= 0) return ND_OK;
  const dim3 grid(static_cast<unsigned>(a.n_samples), static_cast<unsigned>((2 * a.hidden + 127) / 128));
  NormArgs copy = a;
  return launch_checked(reinterpret_cast<const void*>(norm_dparam_stage2_kernel), 0, 128, copy, 0, st, grid);
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
                    int64_t seq_len, int64_t hidden, float eps, void* stream, const float* q_scale = nullptr,
                    float* q_amax = nullptr) {
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
  a.q_scale = q_scale; a.q_amax = q_amax;
  return dispatch(dtype, a, stream);
}

int gated_residual_fwd_any(int dtype, const void* x, const void* branch, const void* gate, void* y, int64_t rows,
                           int64_t row_start, int64_t seq_len, int64_t hidden, void* stream);  // rowops.cu

// Forward with the gated residual in front: x_new = x + gate[b] * branch (gate null: x + branch), then the norm of
// x_new. One kernel where the bulk-copy kernels apply, else the residual kernel followed by the norm kernel
// (identical results: both round x_new once and normalise the rounded values).
static int norm_fwd_residual(bool rms, int dtype, const void* x, const void* branch, const void* gate, const void* scale,
                             const void* shift, void* x_new, void* y, float* mean, float* invstd, int64_t rows,
                             int64_t row_start, int64_t seq_len, int64_t hidden, float eps, void* stream) {
  if (int s = check_shape(rows, row_start, seq_len, hidden)) return s;
  if (rows == 0) return ND_OK;
  if (!x || !branch || !scale || !shift || !x_new || !y) return ND_ERR_BAD_ARG;
  if (!rms && ((mean == nullptr) != (invstd == nullptr))) return ND_ERR_BAD_ARG;
  NormArgs a{};
  a.x = x; a.dy = branch; a.gate = gate; a.dx = x_new; a.res = true;
  a.scale = scale; a.shift = shift; a.y = y;
  a.mean = rms ? nullptr : mean;
  a.invstd = invstd;
  a.rows = rows; a.row_start = row_start;
  a.seq_len = static_cast<int>(seq_len); a.hidden = static_cast<int>(hidden);
  a.eps = eps; a.mode = kFwd; a.rms = rms;
  const int s = dispatch(dtype, a, stream);
  if (s != ND_ERR_UNSUPPORTED) return s;
  if (int r = gated_residual_fwd_any(dtype, x, branch, gate, x_new, rows, row_start, seq_len, hidden, stream)) return r;
  return norm_fwd(rms, dtype, x_new, scale, shift, y, mean, invstd, rows, row_start, seq_len, hidden, eps, stream);
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
    if (!ws || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u)) return ND_ERR_WORKSPACE;
    a.ws_part = static_cast<float*>(ws);
  }
  return dispatch(dtype, a, stream);
}

}  // namespace nd

using namespace nd;

extern "C" {

// Tuning hook used by the benchmark sweeps: force the row-tile height of the
// norm kernels (0 restores the built-in choice). Process-wide.
void nd_tune_norm_tile_rows(int tile_rows) { g_tile_rows_override.store(tile_rows < 0 ? 0 : tile_rows); }

// Tuning hook: 0 = default; 1 = the generic (register-fed) kernels even where the bulk-copy kernels apply;
// 3 / 4 = never / always use the warp-per-row forward kernel where it applies (default: large tensors only);
// 5 = cut the rows evenly even where whole samples would allow sample-aligned chunks. Process-wide.
void nd_tune_norm_variant(int variant) { g_norm_variant.store(variant); }
// Tuning hook: shared-memory pipeline depth of the bulk-copy norm kernels (0 = as many as fit).
void nd_tune_norm_stages(int stages) { g_norm_stages.store(stages < 0 ? 0 : stages); }
// Tuning hook: 0 launches the norm kernels without programmatic stream serialization (default 1).
void nd_tune_norm_pdl(int enabled) { g_norm_pdl.store(enabled != 0); }
// Test hook for the abort path of the bulk-copy norm kernels: `limit_ns` bounds every wait on a copy (0 restores
// the 1 s default); `withhold_first_copy` != 0 makes CTA 0 leave its first copy unsent, so that its first wait
// runs out with nothing in flight, the device error word is set and the CTA returns through the abort path.
void nd_tune_norm_wait_test(unsigned long long limit_ns, int withhold_first_copy) {
  g_norm_wait_limit_ns.store(limit_ns == 0 ? 1000000000ull : limit_ns);
  g_norm_withhold.store(withhold_first_copy != 0);
}
// Tuning hook: cap on CTAs per SM of the bulk-copy norm kernels (0 = what occupancy allows).
void nd_tune_norm_chunks_per_sm(int n) { g_norm_cps.store(n < 0 ? 0 : n); }

size_t nd_norm_dparam_ws_bytes(int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden) {
  if (check_shape(rows, row_start, seq_len, hidden) != ND_OK || rows == 0) return 0;
  return partial_slots(rows, row_start, seq_len) * 2 * static_cast<size_t>(hidden) * sizeof(float);
}

int nd_adaln_fwd(int dtype, const void* x, const void* scale, const void* shift, void* y,
                 float* mean, float* invstd, int64_t rows, int64_t row_start, int64_t seq_len,
                 int64_t hidden, float eps, void* stream) {
  return norm_fwd(false, dtype, x, scale, shift, y, mean, invstd, rows, row_start, seq_len, hidden,
                  eps, stream);
}

// Forward with FP8 e4m3 output for an FP8 consumer (FC1): q = saturate_e4m3(y / *q_scale) and, when `amax` is given,
// *amax = max(*amax, max |y|) - the caller derives the next step's scale from it (delayed scaling) and zeroes it
// when it wants a fresh maximum. Rows up to 192 16-byte vectors wide (H <= 1536 for 16-bit inputs).
int nd_adaln_fwd_e4m3(int dtype, const void* x, const void* scale, const void* shift, void* q, float* mean,
                      float* invstd, const float* q_scale, float* amax, int64_t rows, int64_t row_start,
                      int64_t seq_len, int64_t hidden, float eps, void* stream) {
  if (!q_scale) return ND_ERR_BAD_ARG;
  return norm_fwd(false, dtype, x, scale, shift, q, mean, invstd, rows, row_start, seq_len, hidden, eps, stream,
                  q_scale, amax);
}

int nd_adarms_fwd_e4m3(int dtype, const void* x, const void* scale, const void* shift, void* q, float* inv_rms,
                       const float* q_scale, float* amax, int64_t rows, int64_t row_start, int64_t seq_len,
                       int64_t hidden, float eps, void* stream) {
  if (!q_scale) return ND_ERR_BAD_ARG;
  return norm_fwd(true, dtype, x, scale, shift, q, nullptr, inv_rms, rows, row_start, seq_len, hidden, eps, stream,
                  q_scale, amax);
}

int nd_adaln_fwd_residual(int dtype, const void* x, const void* branch, const void* gate, const void* scale,
                          const void* shift, void* x_new, void* y, float* mean, float* invstd, int64_t rows,
                          int64_t row_start, int64_t seq_len, int64_t hidden, float eps, void* stream) {
  return norm_fwd_residual(false, dtype, x, branch, gate, scale, shift, x_new, y, mean, invstd, rows, row_start,
                           seq_len, hidden, eps, stream);
}

int nd_adarms_fwd_residual(int dtype, const void* x, const void* branch, const void* gate, const void* scale,
                           const void* shift, void* x_new, void* y, float* inv_rms, int64_t rows, int64_t row_start,
                           int64_t seq_len, int64_t hidden, float eps, void* stream) {
  return norm_fwd_residual(true, dtype, x, branch, gate, scale, shift, x_new, y, nullptr, inv_rms, rows, row_start,
                           seq_len, hidden, eps, stream);
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
