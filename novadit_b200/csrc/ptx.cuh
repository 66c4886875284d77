// Thin wrappers over the PTX the kernels share: shared-memory addresses, mbarriers, the
// nanosecond timer used to bound every wait, and 1-D bulk (TMA) copies.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace nd {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}


// 1-D bulk copy global -> shared, completion counted in bytes on `bar`. Both addresses 16-byte
// aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Programmatic dependent launch. A kernel launched with the programmatic-serialization attribute may
// start while its predecessor in the stream is still running; `griddep_wait` blocks until that
// predecessor has completed and its writes are visible, so it must precede the first read of any
// global input. `griddep_launch_dependents` lets the successor start early. Both are no-ops for a
// kernel launched without the attribute.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy
// (bulk copy) accesses.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Wait on an mbarrier phase for at most one second (`limit_ns`: a test may shorten it). Returns false (and
// records `code` in the device error word `err`, read on the host with nd_device_error()) on expiry.
__device__ __forceinline__ bool mbar_wait_1s(uint64_t* bar, uint32_t parity, int* err, int code,
                                             unsigned long long limit_ns = 1000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t polls = 1;; ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 1023u) == 0 && global_ns() - t0 > limit_ns) {
      if (err != nullptr) atomicCAS(err, 0, code);
      return false;
    }
  }
}

}  // namespace nd
