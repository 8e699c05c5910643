// Launch table of the single-query (suffix) kernel for block size 16, the size ParrotServe's vLLM-layout
// engine configurations use; the kernel itself is in single_query.cuh.
#include "single_query.cuh"

namespace pb {

cudaError_t launch_single_query(const AttnDev& d, int dtype, int head_size, int block_size, cudaStream_t s) {
  // block sizes 8 and 32 (the reference dispatches 8 / 16 / 32, csrc/attention/attention_kernels.cu:504-524):
  // the fp32-FMA consumer, compiled in files of their own
  if (block_size == 8) return launch_single_query_b8(d, dtype, head_size, s);
  if (block_size == 32) return launch_single_query_b32(d, dtype, head_size, s);
  if (head_size == 128 && block_size == 16) {
    if (dtype == PB_F16) return launch_sq<__half, 128, 16, 8, 3, true>(d, s);
    if (dtype == PB_BF16) return launch_sq<__nv_bfloat16, 128, 16, 8, 3, true>(d, s);
    if (dtype == PB_F32) return launch_sq<float, 128, 16, 4, 3, false>(d, s);
  }
  if (head_size == 64 && block_size == 16) {
    if (dtype == PB_F16) return launch_sq<__half, 64, 16, 8, 4, true>(d, s);
    if (dtype == PB_BF16) return launch_sq<__nv_bfloat16, 64, 16, 8, 4, true>(d, s);
    if (dtype == PB_F32) return launch_sq<float, 64, 16, 8, 3, false>(d, s);
  }
  // The other head sizes of the reference's paged-attention kernels (csrc/attention/attention_kernels.cu:457-478:
  // 64, 80, 96, 112, 128, 256): same kernel, warps and stages chosen to fit shared memory.
#define PB_SQ_HEAD(DD, W16, W32)                                                              \
  if (head_size == DD && block_size == 16) {                                                  \
    if (dtype == PB_F16) return launch_sq<__half, DD, 16, W16, 3, true>(d, s);                \
    if (dtype == PB_BF16) return launch_sq<__nv_bfloat16, DD, 16, W16, 3, true>(d, s);        \
    if (dtype == PB_F32) return launch_sq<float, DD, 16, W32, 3, false>(d, s);                \
  }
  PB_SQ_HEAD(80, 8, 6)
  PB_SQ_HEAD(96, 8, 5)
  PB_SQ_HEAD(112, 8, 4)
  PB_SQ_HEAD(256, 4, 2)
#undef PB_SQ_HEAD
  return cudaErrorInvalidValue;
}

}  // namespace pb
