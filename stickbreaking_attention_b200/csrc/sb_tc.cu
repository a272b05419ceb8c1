// Tensor-core (tcgen05 + TMEM + TMA) kernels.  Placeholder until the kernels land.
#include "sb_common.cuh"

namespace sb {
bool tc_supported(int, int) { return false; }
cudaError_t launch_tc_fwd(const KParams &, int, cudaStream_t, int *) { return cudaErrorNotSupported; }
cudaError_t launch_tc_bwd(const KParams &, int, cudaStream_t, int *) { return cudaErrorNotSupported; }
}  // namespace sb
