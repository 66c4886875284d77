// Host-side selection and launch of the AdaLN / AdaRMSNorm kernels.
//
// Rows that are 16-byte vectorisable and at most 512 vectors wide (H <= 4096 for 16-bit types)
// take the bulk-copy kernels of norm_tma.cuh: one balanced wave of CTAs, one chunk of rows each.
// Everything else (ragged or misaligned rows, very wide rows) takes the generic kernels of
// norm_impl.cuh, which cut the rows into (sample, tile) items. A backward launch that produces
// dscale/dshift is followed by the small stage-2 kernel that sums the fp32 partials.
#pragma once

#include "norm_tma.cuh"

namespace nd {

int norm_stages_override();  // tuning: pipeline depth of the bulk-copy kernels (0 = by budget)

inline int launch_checked(const void* fn, long long grid, int nt, NormArgs& a, int smem, cudaStream_t st) {
  void* params[] = {&a};
  cudaError_t e = cudaLaunchKernel(fn, dim3(static_cast<unsigned>(grid)), dim3(nt), params, smem, st);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return ND_ERR_LAUNCH;
  }
  return ND_OK;
}

inline long long resident_slots(const void* fn, int nt, int smem) {
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, nt, smem) != cudaSuccess || occ < 1) {
    (void)cudaGetLastError();
    occ = 1;
  }
  if (occ > kMaxChunksPerSm) occ = kMaxChunksPerSm;  // the workspace is sized for this many CTAs per SM
  return static_cast<long long>(occ) * sm_count();
}

template <typename T, int VEC>
int launch_norm_tma(NormArgs a, cudaStream_t st) {
  constexpr int RPI = 4;
  const int nvec = a.hidden / VEC;
  const int nt = (nvec + 31) / 32 * 32;
  const void* fn = pick_tma<T, VEC, RPI, 96, 136>(a.mode, a.rms);
  // as many pipeline stages as fit the per-CTA shared-memory budget (4 forward / 3 backward CTAs per SM)
  const int tensors = a.mode == kFwd ? 1 : 2;
  const int stage_bytes = tensors * RPI * a.hidden * static_cast<int>(sizeof(T));
  const int budget = a.mode == kFwd ? 54 * 1024 : 72 * 1024;
  int stages = norm_stages_override() > 0 ? norm_stages_override() : budget / stage_bytes;
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
  long long chunks = resident_slots(fn, nt, smem);
  const long long most = a.rows / RPI > 1 ? a.rows / RPI : 1;  // every chunk holds at least one full group
  if (chunks > most) chunks = most;
  a.n_chunks = static_cast<int>(chunks);
  a.b_first = a.row_start / a.seq_len;
  a.n_samples = (a.row_start + a.rows - 1) / a.seq_len - a.b_first + 1;
  if (int s = launch_checked(fn, chunks, nt, a, smem, st)) return s;
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
  const void* ptrs[] = {a.x, a.scale, a.shift, a.y, a.dy, a.dx, a.dscale, a.dshift, a.ws_part};
  for (const void* p : ptrs) vec_ok = vec_ok && aligned16(p);
  a.err = device_error_ptr();
  if (!vec_ok) return launch_norm_generic<T, 1>(a, st);
  if (a.hidden / VMAX <= 512 && norm_variant() != 1) return launch_norm_tma<T, VMAX>(a, st);
  return launch_norm_generic<T, VMAX>(a, st);
}

}  // namespace nd
