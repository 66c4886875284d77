// AdaLN / AdaRMSNorm kernels instantiated for float rows.
#include "norm_launch.cuh"

namespace nd {
int launch_norm_f32(const NormArgs& a, cudaStream_t st) { return launch_norm<float>(a, st); }
}  // namespace nd
