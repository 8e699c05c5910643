/*
 * parrot_b200_attn.h — C ABI of the B200 (sm_100a) shared-prefix paged attention library.
 *
 * The library replaces the native ops behind ParrotServe's builtin-engine attention path:
 *   - `parrot.attention_ops`  (csrc/attention.cpp:4-62, kernels in csrc/attention/*.cu)
 *   - `vllm.cache_ops`        (3rdparty/vllm/csrc/cache.cpp:6-46, cache_kernels.cu)
 *   - the Triton kernels in parrot/engine/builtin/kernels/{shared_flash_decoding,tokens_moving}.py
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless said otherwise.
 *   - Every function enqueues work on `stream` (a cudaStream_t passed as void*), never
 *     synchronises the host and never allocates, except pb_read_status (which synchronises
 *     the stream so that it can read the status word).
 *   - Return value: 0 (PB_OK) or a negative pb_status. Nothing throws across this ABI.
 *   - Paged KV cache layout (parrot/engine/builtin/mem.py:69-82):
 *       K: [num_blocks, num_kv_heads, head_size/x, block_size, x]   x = 16 / sizeof(element)
 *       V: [num_blocks, num_kv_heads, head_size, block_size]
 *     A slot s addresses block s / block_size, offset s % block_size.
 *   - Softmax statistics exchanged through `qk_max` / `exp_sum` use the reference's base-2
 *     convention (csrc/attention/attention_post_kernels.cu:147,321-340): qk_max is the row
 *     maximum of q.k * scale * log2(e), exp_sum = sum 2^(logit - qk_max), and `out` holds the
 *     NORMALISED partial output.
 */
#ifndef PARROT_B200_ATTN_H_
#define PARROT_B200_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pb_dtype { PB_F32 = 0, PB_F16 = 1, PB_BF16 = 2 } pb_dtype;

typedef enum pb_status {
  PB_OK = 0,
  PB_ERR_INVALID_ARG = -1,   /* null pointer, negative size, misaligned pointer/stride      */
  PB_ERR_UNSUPPORTED = -2,   /* head_size / block_size / dtype outside the compiled set     */
  PB_ERR_WORKSPACE = -3,     /* workspace missing or smaller than pb_attn_workspace_bytes   */
  PB_ERR_LAUNCH = -4,        /* the CUDA runtime refused a launch (see pb_last_cuda_error)  */
  PB_ERR_DEVICE = -5         /* a kernel recorded a fault in the workspace status word      */
} pb_status;

/* Stats handling of one attention call (the prev/post split of csrc/attention.cpp:19-47). */
typedef enum pb_stats_mode {
  PB_STATS_NONE = 0,   /* final output only                                                  */
  PB_STATS_SAVE = 1,   /* also write qk_max / exp_sum of everything this call attended       */
  PB_STATS_LOAD = 2,   /* `out`, qk_max, exp_sum hold an earlier partial: merge it in place  */
  PB_STATS_LOAD_SAVE = 3
} pb_stats_mode;

/*
 * One grouped shared-prefix attention problem over `num_rows` query rows (a decode sequence
 * is one row). Row r attends to   prefix(group of r)  ++  suffix(r).
 *
 * Generalises flash_paged_attention (parrot/engine/builtin/kernels/shared_flash_decoding.py:285-329),
 * which is the case num_groups == 1; num_groups == 0 is plain paged attention
 * (single_query_cached_kv_attention, csrc/attention.cpp:4-17).
 */
typedef struct pb_attn_params {
  /* tensors */
  void* out;                 /* [num_rows, num_heads, head_size], row stride out_stride elements */
  const void* query;         /* [num_rows, num_heads, head_size], row stride q_stride elements   */
  const void* key_cache;
  const void* value_cache;
  const int32_t* head_mapping; /* [num_heads] query head -> kv head, or NULL for identity        */
  float scale;
  int32_t dtype;             /* pb_dtype of query / caches / out                                 */
  int32_t num_rows;
  int32_t num_heads;
  int32_t num_kv_heads;
  int32_t head_size;
  int32_t block_size;
  int64_t num_blocks;        /* physical blocks in the caches (bounds for validation builds)     */
  int64_t q_stride;
  int64_t out_stride;
  int64_t kv_block_stride;   /* elements between physical blocks (same for K and V)              */
  int64_t kv_head_stride;    /* elements between kv heads inside a block                         */
  /* per-row private context ("paged" part) */
  const int32_t* suffix_lens;    /* [num_rows] tokens, may be 0                                  */
  const int32_t* suffix_tables;  /* [num_rows, suffix_table_stride] physical block ids, 0-padded */
  int32_t suffix_table_stride;   /* = max blocks per row; 0 allowed                              */
  /* shared prefixes ("flash" part); rows are sorted by group */
  int32_t num_groups;
  const int32_t* group_row_offsets; /* [num_groups + 1] CSR over rows                            */
  const int32_t* group_prefix_lens; /* [num_groups] tokens (true length, not block padded)       */
  const int32_t* group_tables;      /* [num_groups, group_table_stride] physical block ids       */
  int32_t group_table_stride;
  /* causal segments (prefill requests): rows [seg_row_offsets[s], seg_row_offsets[s+1]) are the new
   * tokens of one request, in order. Row i of a segment of n rows attends, after its group's
   * prefix, the first seg_kv_lens[s] - n + i + 1 tokens of the request's private context
   * (bottom-right aligned causal mask, the mask the reference builds at
   * parrot/engine/builtin/attn_func.py:541-546). Their suffix_lens must be 0. num_segments may be 0. */
  int32_t num_segments;
  const int32_t* seg_row_offsets;   /* [num_segments + 1]                                         */
  const int32_t* seg_kv_lens;       /* [num_segments] private context tokens incl. the new ones   */
  const int32_t* seg_tables;        /* [num_segments, seg_table_stride] physical block ids        */
  int32_t seg_table_stride;
  /* outer prefix groups: a second, independent partition of the rows for a context shared ABOVE the
   * groups (two-level context trees: a system prompt shared by every request, then per-application
   * prompts, then private contexts; the reference's tests build such trees,
   * tests/engine/builtin/test_shared_prefix.py:57-115, but its attention function flattens them to
   * one shared level, parrot/engine/builtin/attn_func.py:411-459). A row attends
   * outer prefix ++ group prefix ++ causal segment ++ private suffix. num_outer_groups may be 0. */
  int32_t num_outer_groups;
  const int32_t* outer_row_offsets; /* [num_outer_groups + 1] CSR over rows                       */
  const int32_t* outer_prefix_lens; /* [num_outer_groups] tokens                                  */
  const int32_t* outer_tables;      /* [num_outer_groups, outer_table_stride] physical block ids  */
  int32_t outer_table_stride;
  /* new tokens of the step, optional (slot_mapping == NULL: none). Every query row is one new token
   * of the iteration (a decode sequence's next token, or one token of a prefill request): row r's
   * key / value are row r of key_new / value_new and belong in cache slot slot_mapping[r] (negative:
   * the row brings no new token). With these fields set the attention call ALSO performs the KV
   * fill (cache_ops.reshape_and_cache, 3rdparty/vllm/csrc/cache_kernels.cu:142-224, which the
   * reference's attention function runs first in every layer, parrot/engine/builtin/attn_func.py:615-621):
   * do not call pb_reshape_and_cache for these tokens. For a pure decode batch without head_mapping
   * there is then no fill launch at all: the warp of the suffix kernel that streams the last block
   * of a row takes the row's new key / value straight from key_new / value_new, puts them where
   * they belong in its copy of the block, and writes them into the cache. That requires a decode
   * row's new token to be the LAST token of its private suffix (suffix_lens counts it), which the
   * planner checks (a mismatch is recorded as a bad index); a batch with causal segments or a
   * head_mapping runs the fill as a kernel of its own before the attention kernels.
   * slot_mapping is read when the work lists are built (pb_attn_plan), key_new / value_new when the
   * attention runs. */
  const void* slot_mapping;    /* [num_rows] int32 (slot_is_i64 == 0) or int64 */
  int32_t slot_is_i64;
  const void* key_new;         /* [num_rows, num_kv_heads, head_size], row stride key_new_stride elements */
  const void* value_new;
  int64_t key_new_stride;
  int64_t value_new_stride;
  /* statistics (base-2 domain), [num_rows, num_heads] fp32; may be NULL for PB_STATS_NONE */
  float* qk_max;
  float* exp_sum;
  int32_t stats_mode;        /* pb_stats_mode                                                    */
  /* tuning; 0 = library default */
  int32_t dense_min_rows;    /* smallest group that takes the tensor-core prefix kernel          */
  int32_t suffix_chunk_blocks;
  int32_t prefix_chunk_blocks;
  int32_t dense_ctas;        /* SMs for the tensor-core prefix kernel; the suffix kernel runs beside it.
                              * Part of the plan: read when the work lists are built */
  int32_t dense_row_tile;    /* query rows per work item of the tensor-core kernel: 128 (one row tile per
                              * pass; shares a row's exponentials between threads when a group has at most
                              * 64 rows) or 256 (two row tiles share every K/V tile, softmax of one under the
                              * MMAs of the other: the prefill shape). 0 = 128.
                              * Part of the plan. Any other value is an invalid argument. */
  /* scratch */
  void* workspace;
  size_t workspace_bytes;
} pb_attn_params;

/* Library/ABI version, bumped on any incompatible change of this header. */
int pb_abi_version(void);

/* Measurement aid, not part of the attention path: two cudaEvent_t handles (or NULL) that the NEXT
 * attention call of the calling thread records on its stream right before and right after its
 * suffix (single-query) kernel, so that a harness can time that kernel inside its own timed
 * region. The request is consumed by that call. */
void pb_attn_set_timing_events(void* begin, void* end);

/* Text of the last CUDA runtime error seen by this library on the calling thread. */
const char* pb_last_cuda_error(void);

/* Bytes of scratch pb_shared_prefix_attention needs for these static bounds. Only the sizes,
 * strides, num_groups and tuning fields of `p` are read. Returns 0 on invalid sizes. */
size_t pb_attn_workspace_bytes(const pb_attn_params* p);

/* Builds the per-iteration work lists (device-side, from the device-resident lengths) into the
 * workspace. The lists depend only on lengths/tables, not on the layer: build once per
 * iteration, run pb_shared_prefix_attention_planned once per layer. */
int pb_attn_plan(const pb_attn_params* p, void* stream);

/* Attention over an already planned workspace (prefix stage and suffix stage side by side, then
 * the merge). If a kernel of the call recorded a fault in the workspace status word
 * (pb_read_status), the merge overwrites the call's whole output with NaN. */
int pb_shared_prefix_attention_planned(const pb_attn_params* p, void* stream);

/* pb_attn_plan + pb_shared_prefix_attention_planned.
 * Replaces flash_paged_attention / paged_flash_attention
 * (parrot/engine/builtin/kernels/shared_flash_decoding.py:285-376). */
int pb_shared_prefix_attention(const pb_attn_params* p, void* stream);

/* Synchronises `stream`, returns PB_OK or PB_ERR_DEVICE if a kernel recorded a bounded-wait
 * expiry or an out-of-range index in this workspace; *detail (optional, host) gets the raw word. */
int pb_read_status(const void* workspace, void* stream, int32_t* detail);

/*
 * The three entry points of `parrot.attention_ops` (csrc/attention.cpp:4-47), with the tensors
 * flattened to pointers and strides. Of the two extra tensors of the 13-argument plain form the
 * reference kernel never reads `block_lens` and walks `block_nums[seq]` table entries, masking
 * tokens at or beyond `context_lens[seq]` (csrc/attention/attention_kernels.cu:159-162,203);
 * this library walks ceil(context_len / block_size) blocks, the same attention for every
 * consistent block_nums, so a torch shim accepts both tensors and drops them.
 *   plain: out = attention over block_tables/context_lens.
 *   prev : same, and writes qk_maxs / exp_sums            (attention_prev_kernels.cu:331-337).
 *   post : same, merged in place with the partial result already in out / prev_qk_maxs /
 *          prev_exp_sums                                   (attention_post_kernels.cu:321-340).
 * alibi slopes are not supported (the reference always passes None).
 */
int pb_single_query_cached_kv_attention(
    void* out, const void* query, const void* key_cache, const void* value_cache,
    const int32_t* head_mapping, float scale, const int32_t* block_tables,
    const int32_t* context_lens, int32_t block_size, int32_t max_context_len,
    int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads, int32_t head_size,
    int32_t max_num_blocks_per_seq, int64_t q_stride, int64_t kv_block_stride,
    int64_t kv_head_stride, int64_t num_blocks, int32_t dtype, void* workspace,
    size_t workspace_bytes, void* stream);

int pb_single_query_cached_kv_prev_attention(
    void* out, const void* query, const void* key_cache, const void* value_cache,
    const int32_t* head_mapping, float scale, const int32_t* block_tables,
    const int32_t* context_lens, float* qk_maxs, float* exp_sums, int32_t block_size,
    int32_t max_context_len, int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads,
    int32_t head_size, int32_t max_num_blocks_per_seq, int64_t q_stride,
    int64_t kv_block_stride, int64_t kv_head_stride, int64_t num_blocks, int32_t dtype,
    void* workspace, size_t workspace_bytes, void* stream);

int pb_single_query_cached_kv_post_attention(
    void* out, const void* query, const void* key_cache, const void* value_cache,
    const int32_t* head_mapping, float scale, const int32_t* block_tables,
    const int32_t* context_lens, float* prev_qk_maxs, float* prev_exp_sums,
    int32_t block_size, int32_t max_context_len, int32_t num_seqs, int32_t num_heads,
    int32_t num_kv_heads, int32_t head_size, int32_t max_num_blocks_per_seq, int64_t q_stride,
    int64_t kv_block_stride, int64_t kv_head_stride, int64_t num_blocks, int32_t dtype,
    void* workspace, size_t workspace_bytes, void* stream);

/*
 * pb_single_query_cached_kv_attention for callers that cannot allocate device memory (a plugin
 * running inside someone else's stream capture, a worker whose memory pool belongs to the engine
 * that loaded it). No counterpart in the reference. The scratch the kernels need lives in a
 * fixed 32 MiB device array inside the library (pb_static_scratch_bytes), so the call takes no
 * workspace and allocates nothing.
 *   - Returns PB_ERR_WORKSPACE when pb_single_query_workspace_bytes(...) for these sizes exceeds
 *     that array: shorten the batch or use the workspace form.
 *   - The first call on a device resolves the array's device address; make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams, different threads) race on it. Serialise them.
 */
int pb_single_query_cached_kv_attention_static(
    void* out, const void* query, const void* key_cache, const void* value_cache,
    const int32_t* head_mapping, float scale, const int32_t* block_tables,
    const int32_t* context_lens, int32_t block_size, int32_t max_context_len,
    int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads, int32_t head_size,
    int32_t max_num_blocks_per_seq, int64_t q_stride, int64_t kv_block_stride,
    int64_t kv_head_stride, int64_t num_blocks, int32_t dtype, void* stream);

/* Size of the library's built-in scratch array. */
size_t pb_static_scratch_bytes(void);

/* pb_read_status for the built-in scratch array of the current device (a caller of the entry point
 * above never sees that array's address): synchronises `stream`, returns PB_OK or PB_ERR_DEVICE;
 * *detail (optional, host) gets the raw status word of the last call that used the array. */
int pb_static_scratch_status(void* stream, int32_t* detail);

/* Workspace bytes for the three functions above. */
size_t pb_single_query_workspace_bytes(int32_t num_seqs, int32_t num_heads, int32_t head_size,
                                       int32_t block_size, int32_t max_num_blocks_per_seq);

/*
 * One attention layer of an iteration for a caller whose tensors live in HOST memory: uploads the
 * step's inputs, writes the new K/V rows into the paged caches, runs the attention and downloads
 * the result, all enqueued on `stream` by this one call (all uploads first, then the kernels). It is the sequence the reference's
 * attention function runs per layer (parrot/engine/builtin/attn_func.py:601-696:
 * vllm_reshape_and_cache at :615, then flash_paged_attention at :684) with the copies a host caller would
 * otherwise issue one by one around it.
 *
 * `p` describes the problem exactly as for pb_shared_prefix_attention; p->query, p->out,
 * p->suffix_lens and p->suffix_tables are DEVICE buffers this call fills from / drains to the host
 * pointers below (query and out must be dense: q_stride == out_stride == num_heads * head_size).
 * Host buffers should be page-locked so that the copies are asynchronous; pageable memory works
 * but makes each copy synchronous. Nothing is allocated.
 */
typedef struct pb_host_step {
  const void* h_query;           /* [num_rows, num_heads, head_size] */
  const void* h_key_new;         /* [num_new_tokens, num_kv_heads, head_size], or NULL: no fill */
  const void* h_value_new;
  const int64_t* h_slot_mapping; /* [num_new_tokens]; negative = skip the token */
  int64_t num_new_tokens;
  const int32_t* h_suffix_lens;   /* [num_rows], or NULL: the device copy is already current */
  const int32_t* h_suffix_tables; /* [num_rows, suffix_table_stride], or NULL likewise */
  void* h_out;                   /* [num_rows, num_heads, head_size] */
  void* d_key_new;               /* device staging for the three fill inputs */
  void* d_value_new;
  int64_t* d_slot_mapping;
  int32_t replan;                /* != 0: rebuild the work lists (lengths or tables changed) */
  int32_t synchronize;           /* != 0: return after the stream has drained (h_out is valid) */
  int32_t merge_adjacent;        /* != 0: the host buffers are parts of ONE page-locked allocation
                                  * and the device buffers parts of one allocation; uploads whose
                                  * host and device ranges follow one another directly are then
                                  * issued as a single transfer (each transfer has a fixed latency
                                  * of several microseconds) */
  int32_t direct_out;            /* != 0: when h_out is page-locked memory the device can address,
                                  * the last kernel writes the result straight into it instead of
                                  * into p->out followed by a download; otherwise ignored */
} pb_host_step;

int pb_attention_step_host(const pb_attn_params* p, const pb_host_step* io, void* stream);

/*
 * KV fill: scatter new key/value rows into the paged caches.
 * Replaces cache_ops.reshape_and_cache (3rdparty/vllm/csrc/cache_kernels.cu:142-224; only call
 * site parrot/engine/builtin/kernels/vllm/reshape_and_cache.py:16).
 *   key/value: [num_tokens, num_heads, head_size] with row strides key_stride / value_stride.
 *   slot_mapping: [num_tokens] int32 (slot_is_i64 == 0) or int64; a negative slot skips the token,
 *   and so does a slot whose block lies outside [0, num_blocks): it is never dereferenced and, as
 *   this entry has no workspace to record it in, not reported either.
 */
int pb_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                         const void* slot_mapping, int32_t slot_is_i64, int64_t num_tokens,
                         int32_t num_heads, int32_t head_size, int32_t block_size,
                         int64_t key_stride, int64_t value_stride, int64_t kv_block_stride,
                         int64_t kv_head_stride, int64_t num_blocks, int32_t dtype, void* stream);

/*
 * NeoX rotary embedding of q and k fused with the KV fill: one pass over q, k and v instead of the
 * reference's rotary kernel (read + write q and k) followed by reshape_and_cache (read k and v again).
 * Replaces pos_encoding_ops.rotary_embedding_neox (3rdparty/vllm/csrc/pos_encoding_kernels.cu:7-92;
 * call site parrot/engine/builtin/models/llama.py:123-129 via kernels/vllm/rotary_embed.py:10-25)
 * followed by cache_ops.reshape_and_cache (3rdparty/vllm/csrc/cache_kernels.cu:142-224).
 *   query [num_tokens, num_heads, head_size] is rotated IN PLACE; the rotated key row goes into its
 *   cache cell and is written back into `key` only when write_key_back != 0; value is cached as is.
 *   positions [num_tokens] int64 (clamped to [0, max_position)); cos_sin_cache [max_position, rot_dim]
 *   of the tensors' dtype, each row = cos(rot_dim/2) then sin(rot_dim/2). The first rot_dim elements
 *   of every head are rotated (x = d, y = d + rot_dim/2), the rest pass through. rot_dim must be a
 *   multiple of 2 * (16 / sizeof(element)). Products are formed in fp32 and rounded once.
 *   key_cache == NULL: rotation only (q and k in place), exactly the reference's rotary call;
 *   value, value_cache and slot_mapping are then ignored.
 */
int pb_rotary_reshape_and_cache(void* query, void* key, const void* value, void* key_cache, void* value_cache,
                                const void* slot_mapping, int32_t slot_is_i64, const int64_t* positions,
                                const void* cos_sin_cache, int32_t rot_dim, int64_t max_position, int64_t num_tokens,
                                int32_t num_heads, int32_t num_kv_heads, int32_t head_size, int32_t block_size,
                                int64_t query_stride, int64_t key_stride, int64_t value_stride,
                                int64_t kv_block_stride, int64_t kv_head_stride, int64_t num_blocks,
                                int32_t write_key_back, int32_t dtype, void* stream);

/* Inverse of pb_reshape_and_cache (paged -> [num_tokens, num_heads, head_size]).
 * Replaces cache_ops.gather_cached_kv (3rdparty/vllm/csrc/cache_kernels.cu:229-386). */
int pb_gather_cached_kv(void* key, void* value, const void* key_cache, const void* value_cache,
                        const void* slot_mapping, int32_t slot_is_i64, int64_t num_tokens,
                        int32_t num_heads, int32_t head_size, int32_t block_size,
                        int64_t key_stride, int64_t value_stride, int64_t kv_block_stride,
                        int64_t kv_head_stride, int64_t num_blocks, int32_t dtype, void* stream);

/* dest[dest_indices[i]] = K (is_value == 0) or V (is_value != 0) row at slot src_slots[i].
 * Replaces move_tokens_from_blocked_{k,v}_cache
 * (parrot/engine/builtin/kernels/tokens_moving.py:163-218, 271-313). Indices are int64. */
int pb_move_tokens_from_blocked_cache(const void* cache, void* dest, const int64_t* src_slots,
                                      const int64_t* dest_indices, int64_t num_tokens,
                                      int32_t is_value, int32_t num_heads, int32_t head_size,
                                      int32_t block_size, int64_t dest_stride,
                                      int64_t kv_block_stride, int64_t kv_head_stride,
                                      int64_t num_blocks, int64_t dest_rows, int32_t dtype,
                                      void* stream);

/* dest[dest_indices[i], :] = src[src_indices[i], :] over rows of row_bytes bytes.
 * Replaces discontinuous_move_tokens (parrot/engine/builtin/kernels/tokens_moving.py:67-100). */
int pb_discontinuous_move_tokens(const void* src, void* dest, const int64_t* src_indices,
                                 const int64_t* dest_indices, int64_t num_tokens,
                                 int64_t row_bytes, int64_t src_stride_bytes,
                                 int64_t dest_stride_bytes, int64_t src_rows, int64_t dest_rows,
                                 void* stream);

/*
 * Copies whole cache blocks inside the K cache and the V cache of every layer (copy-on-write of
 * shared blocks). Replaces cache_ops.copy_blocks (3rdparty/vllm/csrc/cache_kernels.cu:54-138).
 *   key_cache_ptrs / value_cache_ptrs: DEVICE arrays [num_layers] of cache base addresses;
 *   block_pairs: DEVICE array [num_pairs][2] of (source block, destination block); a pair with a
 *   block outside [0, num_blocks) is skipped; block_bytes = bytes of one block of one cache
 *   (num_kv_heads * head_size * block_size * sizeof(element)), a multiple of 16.
 */
int pb_copy_blocks(const int64_t* key_cache_ptrs, const int64_t* value_cache_ptrs, int32_t num_layers,
                   const int64_t* block_pairs, int64_t num_pairs, int64_t block_bytes, int64_t num_blocks,
                   void* stream);

/*
 * Copies cache blocks between two caches of the same block size: direction 0 device -> device,
 * 1 device -> host, 2 host -> device. Replaces cache_ops.swap_blocks
 * (3rdparty/vllm/csrc/cache_kernels.cu:9-50). host_block_pairs: HOST array [num_pairs][2] of
 * (source block, destination block), checked against src_blocks / dst_blocks before anything is
 * enqueued; runs of pairs with consecutive source AND destination blocks go out as one copy.
 */
int pb_swap_blocks(const void* src, void* dst, const int64_t* host_block_pairs, int64_t num_pairs,
                   int64_t block_bytes, int64_t src_blocks, int64_t dst_blocks, int32_t direction, void* stream);

/*
 * Draws one token per row of a [num_rows, vocab] logits matrix: logits / temperature, nucleus
 * (top-p) filtering, softmax, one draw. Replaces the part of Sampler.forward after the logits GEMM
 * (parrot/engine/builtin/models/sampler.py:33-66): a token is dropped when the probability mass of
 * the tokens sorted before it (descending logit, ties by index) exceeds top_p, exactly the mask the
 * reference builds from its sorted cumulative sum; the row is never sorted here.
 *   logits: DEVICE [num_rows][row_stride] elements of `dtype` (pb_dtype), row_stride >= vocab;
 *   temperature, top_p: DEVICE [num_rows] floats, or NULL for 1.0 (temperature must be > 0);
 *   uniforms: DEVICE [num_rows] floats in [0, 1): the draw is the inverse CDF over the kept tokens in
 *   index order, so one call is a pure function of its inputs and repeats bit for bit;
 *   ids: DEVICE [num_rows] int64 token ids (the reference returns int64).
 */
int pb_sample_top_p(const void* logits, int32_t dtype, int32_t num_rows, int32_t vocab, int64_t row_stride,
                    const float* temperature, const float* top_p, const float* uniforms, int64_t* ids,
                    void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PARROT_B200_ATTN_H_ */
