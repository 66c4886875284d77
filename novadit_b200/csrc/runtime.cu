// Process-wide helpers of the C ABI: status strings, last CUDA error, device facts.
#include "common.cuh"
#include "ptx.cuh"

namespace nd {

__device__ int g_device_error = 0;  // set by a kernel whose bounded wait expired

static thread_local int t_last_cuda_error = 0;

void set_last_cuda_error(cudaError_t e) { t_last_cuda_error = static_cast<int>(e); }

// Device address of the error word of the current device (nullptr if it cannot be resolved).
int* device_error_ptr() {
  constexpr int kMaxDevices = 64;
  static int* cache[kMaxDevices] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return nullptr;
  }
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_error) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cache[dev] = static_cast<int*>(p);
  }
  return cache[dev];
}

int sm_count() {
  constexpr int kMaxDevices = 64;
  static int cache[kMaxDevices] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return 148;
  }
  if (cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = 148;
    }
    cache[dev] = n;
  }
  return cache[dev];
}

}  // namespace nd

extern "C" {

const char* nd_status_string(int status) {
  switch (status) {
    case ND_OK: return "ok";
    case ND_ERR_BAD_ARG: return "bad argument (null pointer, negative size or inconsistent shape)";
    case ND_ERR_UNSUPPORTED: return "unsupported element type or size";
    case ND_ERR_LAUNCH: return "CUDA launch failed";
    case ND_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
    case ND_ERR_DEVICE: return "a bounded device-side wait expired";
    case ND_ERR_TOO_LARGE: return "problem too large for the built-in scratch of the no-allocation entry point";
    default: return "unknown status";
  }
}

int nd_last_cuda_error(void) { return nd::t_last_cuda_error; }

int nd_version(void) { return 100; }

int nd_device_error(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, nd::g_device_error, sizeof(int)) != cudaSuccess) {
    nd::set_last_cuda_error(cudaGetLastError());
    return ND_ERR_LAUNCH;
  }
  if (reset && v != 0) {
    const int zero = 0;
    (void)cudaMemcpyToSymbol(nd::g_device_error, &zero, sizeof(int));
  }
  return v;
}

}  // extern "C"
