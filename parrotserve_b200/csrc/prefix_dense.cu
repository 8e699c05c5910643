// Dense shared-prefix stage (tensor cores). Placeholder until the tcgen05 kernel lands: reports
// "no dense path", so the planner routes every prefix through the single-query kernel.
#include "common.cuh"

namespace pb {

bool dense_prefix_supported(int, int, int) { return false; }

cudaError_t launch_dense_prefix(const AttnDev&, int, int, int, cudaStream_t) { return cudaErrorNotSupported; }

}  // namespace pb
