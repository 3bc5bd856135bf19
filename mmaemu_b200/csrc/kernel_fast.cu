// Placeholder until the fast kernel lands: nothing is supported, so every request runs on the integer kernel.
#include "common.cuh"

namespace mmb {
bool fast_supports(const Params&, int) { return false; }
cudaError_t launch_fast(const Params&, int, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace mmb
