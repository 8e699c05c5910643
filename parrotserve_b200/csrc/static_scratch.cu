// Paged decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a plugin invoked while the
// embedding runtime is capturing or replaying work, a sandboxed worker whose memory pool is owned
// and fully handed out by the engine that loaded it, or a callback that may not touch the
// allocator at all. For them the scratch that the attention kernels need (work lists and
// per-chunk partial results) lives in a fixed device array that is part of the loaded module, so
// nothing is allocated at call time. The price is a hard size limit and one shared buffer.
#include <mutex>

#include "common.cuh"

namespace pb {
namespace {

constexpr size_t kStaticScratchBytes = size_t(32) << 20;  // 32 MiB, held by every GPU that loads the library

// Module-scope device storage. In HOST code this name is only a handle for the runtime's symbol
// calls; it is not a device address and must never be passed to a kernel directly.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the CURRENT device; resolved once per device.
int static_scratch_ptr(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_cuda_error(e); return PB_ERR_LAUNCH; }
  if (dev < 0 || dev >= kMaxDevices) return PB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) { set_cuda_error(e); return PB_ERR_LAUNCH; }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return PB_OK;
}

}  // namespace
}  // namespace pb

extern "C" {

size_t pb_static_scratch_bytes(void) { return pb::kStaticScratchBytes; }

int pb_single_query_cached_kv_attention_static(
    void* out, const void* query, const void* key_cache, const void* value_cache,
    const int32_t* head_mapping, float scale, const int32_t* block_tables, const int32_t* context_lens,
    int32_t block_size, int32_t max_context_len, int32_t num_seqs, int32_t num_heads,
    int32_t num_kv_heads, int32_t head_size, int32_t max_num_blocks_per_seq, int64_t q_stride,
    int64_t kv_block_stride, int64_t kv_head_stride, int64_t num_blocks, int32_t dtype, void* stream) {
  const size_t need = pb_single_query_workspace_bytes(num_seqs, num_heads, head_size, block_size, max_num_blocks_per_seq);
  if (need == 0) return PB_ERR_UNSUPPORTED;
  if (need > pb::kStaticScratchBytes) return PB_ERR_WORKSPACE;  // problem too large for the fixed scratch
  void* scratch = nullptr;
  const int rc = pb::static_scratch_ptr(&scratch);
  if (rc != PB_OK) return rc;
  // The array keeps whatever the previous call left behind; nothing of it is read before it is
  // written: the planner kernel of this call starts by resetting the header (status word, work
  // counter) and rebuilds every list the later kernels read.
  return pb_single_query_cached_kv_attention(out, query, key_cache, value_cache, head_mapping, scale, block_tables,
                                             context_lens, block_size, max_context_len, num_seqs, num_heads,
                                             num_kv_heads, head_size, max_num_blocks_per_seq, q_stride,
                                             kv_block_stride, kv_head_stride, num_blocks, dtype, scratch,
                                             pb::kStaticScratchBytes, stream);
}

int pb_static_scratch_status(void* stream, int32_t* detail) {
  void* scratch = nullptr;
  const int rc = pb::static_scratch_ptr(&scratch);
  if (rc != PB_OK) return rc;
  return pb_read_status(scratch, stream, detail);
}

}  // extern "C"
