// nd_adaln_bwd_noalloc: the one-pass AdaLN backward for callers that cannot hand over scratch memory.
//
// Some hosts of this library have no way to allocate device memory when they call it: a serving
// process that gave every free byte to its own pool at start-up, a plugin whose host forbids
// allocations by the libraries it loads, or any code running where cudaMalloc is illegal or would
// stall the whole device (inside a stream capture, inside a latency-critical loop). For them the
// scratch of the dparam reduction lives in the library image itself: a fixed array in device
// global memory that every GPU which loads the library holds until the process exits.
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t kScratchBytes = 16u << 20;  // 16 MiB: covers the DiT-XL/2 shapes (11.3 MB at H = 1152)

// The scratch itself. In host code this name is only a handle for the runtime, not an address a
// kernel could use: the device address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_lock;
void* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch on the CURRENT device; resolved on first use per device.
int scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    nd::set_last_cuda_error(e);
    return ND_ERR_LAUNCH;
  }
  if (dev < 0 || dev >= kMaxDevices) return ND_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> guard(g_lock);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_scratch);  // with device `dev` current: the address is per device
    if (e != cudaSuccess || p == nullptr) {
      nd::set_last_cuda_error(e);
      (void)cudaGetLastError();
      return ND_ERR_LAUNCH;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return ND_OK;
}

}  // namespace

extern "C" {

size_t nd_noalloc_scratch_bytes(void) { return kScratchBytes; }

int nd_adaln_bwd_noalloc(int dtype, const void* dy, const void* x, const void* scale, const float* mean,
                         const float* invstd, void* dx, float* dscale, float* dshift, int64_t rows,
                         int64_t row_start, int64_t seq_len, int64_t hidden, void* stream) {
  if (rows < 0 || row_start < 0 || seq_len <= 0 || hidden <= 0) return ND_ERR_BAD_ARG;
  if (rows == 0) return ND_OK;
  // Size check first, so that an oversized problem is refused before anything touches the device.
  const size_t need = nd_norm_dparam_ws_bytes(rows, row_start, seq_len, hidden);
  if (need > kScratchBytes) return ND_ERR_TOO_LARGE;
  void* scratch = nullptr;
  if (int s = scratch_address(&scratch)) return s;
  // Same kernels, same order of summation as nd_adaln_bwd; the only difference is whose memory the
  // fp32 partial sums pass through. Nothing in the scratch has to be cleared between calls: every
  // slot a launch reads is written by that launch first.
  return nd_adaln_bwd(dtype, dy, x, scale, mean, invstd, dx, dscale, dshift, rows, row_start, seq_len, hidden,
                      scratch, kScratchBytes, stream);
}

}  // extern "C"
