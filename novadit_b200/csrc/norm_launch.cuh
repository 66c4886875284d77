// Host-side selection and launch of the AdaLN / AdaRMSNorm kernels.
//
// Rows that are 16-byte vectorisable and at most 512 vectors wide (H <= 4096 for 16-bit types)
// take the bulk-copy kernels: one balanced wave of CTAs, one chunk of rows each, one CTA per row group
// (norm_tma.cuh); the forward pass of large tensors with rows up to 192 vectors wide runs one warp per row
// (norm_warp.cuh).
// Everything else (ragged or misaligned rows, very wide rows) takes the generic kernels of
// norm_impl.cuh, which cut the rows into (sample, tile) items. A backward launch that produces
// dscale/dshift is followed by the small stage-2 kernel that sums the fp32 partials.
#pragma once

#include "norm_warp.cuh"

namespace nd {

int norm_stages_override();  // tuning: pipeline depth of the bulk-copy kernels (0 = by budget)

unsigned long long norm_wait_limit_ns();  // tuning / test: limit of the bounded waits (default 1 s)
int norm_withhold_first_copy();           // test: CTA 0 of the bulk-copy kernels leaves its first copy unsent
int norm_pdl_enabled();      // tuning: launch with programmatic stream serialization (default on)
int norm_chunks_per_sm();    // tuning: cap on CTAs per SM for the bulk-copy kernels (0 = occupancy)

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor
// in the stream drains (every norm kernel executes griddepcontrol.wait before its first global read),
// which hides the launch latency between the forward, backward and stage-2 kernels of a step.
inline int launch_checked(const void* fn, long long grid, int nt, NormArgs& a, int smem, cudaStream_t st,
                          dim3 grid3 = dim3(0)) {
  void* params[] = {&a};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid3.x != 0 ? grid3 : dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(nt);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = norm_pdl_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelExC(&cfg, fn, params);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}

inline long long resident_slots(const void* fn, int nt, int smem, bool fwd = true) {
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, nt, smem) != cudaSuccess || occ < 1) {
    (void)cudaGetLastError();
    occ = 1;
  }
  if (occ > kMaxChunksPerSm) occ = kMaxChunksPerSm;  // the workspace is sized for this many CTAs per SM
  const int knob = norm_chunks_per_sm();  // n < 10: cap for both passes; otherwise tens = forward cap, units = backward cap
  const int cap = knob < 10 ? knob : (fwd ? knob / 10 : knob % 10);
  if (cap > 0 && occ > cap) occ = cap;
  return static_cast<long long>(occ) * sm_count();
}

// Cuts the shard into `chunks` chunks (at most one per resident CTA slot). When the shard is whole samples and an
// integral number of chunks per sample fills at least 90 % of the slots, every sample gets that many chunks: no
// chunk crosses a sample boundary, so no CTA pays a second modulation load, a ragged extra row group or a second
// partial slot - at the DiT-XL/2 shape those CTAs (one in fourteen) ended 2 us after the others. Otherwise the
// rows are cut evenly whatever the samples.
inline void plan_chunks(NormArgs& a, long long chunks, int rpi) {
  a.b_first = a.row_start / a.seq_len;
  a.n_samples = (a.row_start + a.rows - 1) / a.seq_len - a.b_first + 1;
  a.chunks_per_sample = 0;
  const bool whole = a.row_start % a.seq_len == 0 && a.rows % a.seq_len == 0;
  const long long k = whole ? chunks / a.n_samples : 0;
  if (norm_variant() != 5 && k >= 1 && a.seq_len / k >= rpi && k * a.n_samples * 10 >= chunks * 9) {
    a.chunks_per_sample = static_cast<int>(k);
    chunks = k * a.n_samples;
  }
  a.n_chunks = static_cast<int>(chunks);
  a.chunk_base = a.rows / chunks;
  a.chunk_rem = static_cast<int>(a.rows % chunks);
}

template <typename T, int VEC, int NV>
static const void* pick_fwd_warp_nv(bool rms, bool q8) {
  if (q8) return rms ? (const void*)norm_fwd_warp<T, VEC, NV, true, true> : (const void*)norm_fwd_warp<T, VEC, NV, false, true>;
  return rms ? (const void*)norm_fwd_warp<T, VEC, NV, true> : (const void*)norm_fwd_warp<T, VEC, NV, false>;
}

// the warp-per-row forward kernel for rows of up to 6 x 32 vectors (H <= 1536 for 16-bit types); null beyond
template <typename T, int VEC>
static const void* pick_fwd_warp(int nvec, bool rms, bool q8 = false) {
  switch ((nvec + 31) / 32) {
    case 1: return pick_fwd_warp_nv<T, VEC, 1>(rms, q8);
    case 2: return pick_fwd_warp_nv<T, VEC, 2>(rms, q8);
    case 3: return pick_fwd_warp_nv<T, VEC, 3>(rms, q8);
    case 4: return pick_fwd_warp_nv<T, VEC, 4>(rms, q8);
    case 5: return pick_fwd_warp_nv<T, VEC, 5>(rms, q8);
    case 6: return pick_fwd_warp_nv<T, VEC, 6>(rms, q8);
    default: return nullptr;
  }
}

// Forward with one warp per row (norm_warp.cuh): 128-thread CTAs, one chunk of rows each, a single wave.
template <typename T, int VEC>
int launch_norm_fwd_warp(NormArgs a, const void* fn, cudaStream_t st) {
  int stages = norm_stages_override() > 0 ? norm_stages_override() : 2;
  if (stages < 2) stages = 2;
  if (stages > kMaxStages) stages = kMaxStages;
  a.stages = stages;
  const int smem = static_cast<int>(norm_warp_smem(a.hidden, static_cast<int>(sizeof(T)), stages));
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  long long chunks = resident_slots(fn, kWarpThreads, smem, true);
  const long long most = a.rows / kWarpRows > 1 ? a.rows / kWarpRows : 1;  // every chunk holds at least one full group
  if (chunks > most) chunks = most;
  plan_chunks(a, chunks, kWarpRows);
  return launch_checked(fn, a.n_chunks, kWarpThreads, a, smem, st);
}

template <typename T, int VEC>
int launch_norm_tma(NormArgs a, cudaStream_t st) {
  if (a.mode == kFwd && a.q_scale != nullptr) {  // e4m3 output exists in the warp-per-row kernel only
    const void* fq = pick_fwd_warp<T, VEC>(a.hidden / VEC, a.rms, true);
    return fq != nullptr ? launch_norm_fwd_warp<T, VEC>(a, fq, st) : ND_ERR_UNSUPPORTED;
  }
  // forward of a large tensor (128 MB and up): one warp per row; measured faster there and slower below
  const bool large = static_cast<double>(a.rows) * a.hidden * sizeof(T) >= 128.0 * 1024 * 1024;
  if (a.mode == kFwd && !a.res && (norm_variant() == 4 || (large && norm_variant() != 3))) {
    if (const void* fw = pick_fwd_warp<T, VEC>(a.hidden / VEC, a.rms)) return launch_norm_fwd_warp<T, VEC>(a, fw, st);
  }
  constexpr int RPI = 4;
  const int nvec = a.hidden / VEC;
  const int nt = (nvec + 31) / 32 * 32;
  // 128 registers per backward thread: three 160-thread CTAs per SM, and 512-thread CTAs still launch
  const void* fn = pick_tma<T, VEC, RPI, 96, 128>(a.mode, a.rms, a.res);
  // as many pipeline stages as fit the per-CTA shared-memory budget (4 forward / 3 backward CTAs per SM; the
  // forward with the residual in front stages two tensors and has the backward's footprint)
  const bool light = a.mode == kFwd && !a.res;
  const int tensors = light ? 1 : 2;
  const int stage_bytes = tensors * RPI * a.hidden * static_cast<int>(sizeof(T));
  // Two stages measured best at the DiT-XL/2 shape: deeper pipelines hold shared memory that the
  // next kernel's CTAs (programmatic dependent launch) could otherwise start in. Never more than fits.
  const int budget = light ? 54 * 1024 : 72 * 1024;
  int stages = norm_stages_override() > 0 ? norm_stages_override() : 2;
  if (stages > budget / stage_bytes) stages = budget / stage_bytes;
  if (stages < 2) stages = 2;
  if (stages > kMaxStages) stages = kMaxStages;
  a.stages = stages;
  const int smem = kBarrierBytes + stages * stage_bytes;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  long long chunks = resident_slots(fn, nt, smem, light);
  const long long most = a.rows / RPI > 1 ? a.rows / RPI : 1;  // every chunk holds at least one full group
  if (chunks > most) chunks = most;
  plan_chunks(a, chunks, RPI);
  // a plan whose chunks each lie inside one sample takes the flat walk in every mode (same resources, same results
  // bit for bit; variant 6 keeps the general kernels)
  if (a.chunks_per_sample > 0 && a.seq_len < (1LL << 30) && norm_variant() != 6) {
    const void* flat = a.mode == kFwd ? pick_tma_flat_fwd<T, VEC, RPI, 96, 128>(a.rms, a.res)
                                      : pick_tma_flat_bwd<T, VEC, RPI, 128>(a.mode, a.rms);
    if (cudaFuncSetAttribute(flat, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess) fn = flat;
    else (void)cudaGetLastError();
  }
  if (int s = launch_checked(fn, a.n_chunks, nt, a, smem, st)) return s;
  return a.mode == kBwdDparam || a.mode == kBwdFused ? launch_dparam_stage2(a, st) : ND_OK;
}

template <typename T, int VEC>
int launch_norm_generic(NormArgs a, cudaStream_t st) {
  const int nvec = a.hidden / VEC;
  const void* fn = nullptr;
  int nt = (nvec + 31) / 32 * 32;
  if (nvec <= 256) {
    fn = pick_kernel<T, VEC, 1, 8, 96, 4, 128>(a.mode, a.rms);
  } else if (nvec <= 512) {
    fn = pick_kernel<T, VEC, 1, 4, 64, 4, 128>(a.mode, a.rms);
  } else if (nvec <= 1024) {
    fn = pick_kernel<T, VEC, 1, 4, 64, 2, 64>(a.mode, a.rms);
  } else if (nvec <= 4096) {
    fn = pick_kernel<T, VEC, 4, 1, 64, 1, 64>(a.mode, a.rms);
    nt = ((nvec + 3) / 4 + 31) / 32 * 32;
  } else {
    return ND_ERR_UNSUPPORTED;
  }
  // tile height: all items in one wave of resident CTAs when the problem is small enough, else tall tiles
  const long long slots = resident_slots(fn, nt, 0);
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
  a.n_chunks = 0;
  a.chunks_per_sample = 0;
  a.b_first = plan.b_first;
  a.n_samples = plan.n_samples;
  a.tile_rows = plan.tile_rows;
  a.tiles_per_sample = plan.tiles_per_sample;
  a.n_items = plan.n_items;
  if (a.n_items == 0) return ND_OK;
  if (int s = launch_checked(fn, a.n_items < slots ? a.n_items : slots, nt, a, 0, st)) return s;
  return a.mode == kBwdDparam || a.mode == kBwdFused ? launch_dparam_stage2(a, st) : ND_OK;
}

template <typename T>
int launch_norm(NormArgs a, cudaStream_t st) {
  constexpr int VMAX = 16 / sizeof(T);
  bool vec_ok = (a.hidden % VMAX) == 0;
  const void* ptrs[] = {a.x, a.scale, a.shift, a.y, a.dy, a.dx, a.dscale, a.dshift, a.ws_part, a.gate};
  for (const void* p : ptrs) vec_ok = vec_ok && aligned16(p);
  a.err = device_error_ptr();
  a.wait_limit_ns = norm_wait_limit_ns();
  a.withhold_first_copy = norm_withhold_first_copy();
  // the residual in front of the norm exists in the bulk-copy kernels only: the caller composes the two operators
  if (a.res && (!vec_ok || a.hidden / VMAX > 512 || norm_variant() == 1)) return ND_ERR_UNSUPPORTED;
  if (!vec_ok) return a.q_scale != nullptr ? ND_ERR_UNSUPPORTED : launch_norm_generic<T, 1>(a, st);
  if (a.q_scale != nullptr && a.hidden / VMAX > 192) return ND_ERR_UNSUPPORTED;
  if (a.q_scale != nullptr || (a.hidden / VMAX <= 512 && norm_variant() != 1)) return launch_norm_tma<T, VMAX>(a, st);
  return launch_norm_generic<T, VMAX>(a, st);
}

}  // namespace nd
