// AdaLN / AdaRMSNorm kernels instantiated for __half rows.
#include "norm_launch.cuh"

namespace nd {
int launch_norm_f16(const NormArgs& a, cudaStream_t st) { return launch_norm<__half>(a, st); }
}  // namespace nd
