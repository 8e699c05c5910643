// Single-query kernel instances for block size 32.
#include "single_query.cuh"

namespace pb {
cudaError_t launch_single_query_b32(const AttnDev& d, int dtype, int head_size, cudaStream_t s) {
  return launch_sq_other_block<32>(d, dtype, head_size, s);
}
}  // namespace pb
