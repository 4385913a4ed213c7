// Placeholder until the tcgen05 kernel lands: reports "not supported" so callers fail loudly.
#include "kernels.cuh"

namespace yahkv {
cudaError_t ConfigurePrefillKernels() { return cudaSuccess; }
cudaError_t LaunchPrefill(const PrefillLaunch&, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace yahkv
