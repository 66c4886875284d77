// AdaLN / AdaRMSNorm kernels instantiated for __nv_bfloat16 rows.
#include "norm_launch.cuh"

namespace nd {
int launch_norm_bf16(const NormArgs& a, cudaStream_t st) { return launch_norm<__nv_bfloat16>(a, st); }
}  // namespace nd
