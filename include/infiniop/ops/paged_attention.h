/*
 * Paged-attention decode: one query token per sequence, GQA/MHA, over a
 * block-table-indexed paged KV cache.  Replaces reference
 * include/infiniop/ops/paged_attention.h:33-91 with identical signatures.
 *
 * Tensors (element strides honoured wherever the reference honours them):
 *   out           [num_seqs, num_heads, value_size]           F16 | BF16
 *   q             [num_seqs, num_heads, head_size]            same dtype
 *   k_cache       [num_blocks, num_kv_heads, block_size, head_size]
 *   v_cache       [num_blocks, num_kv_heads, block_size, value_size]
 *   block_tables  [num_seqs, max_num_blocks_per_seq]          I64 | I32 | U32
 *   seq_lens      [num_seqs]                                  same index dtype
 *   alibi_slopes  [num_heads] F32, optional (descriptor and pointer may be NULL)
 *
 * Token j of sequence i lives at cache[block_tables[i][j / block_size], :, j % block_size, :];
 * q-head h reads kv-head h / (num_heads / num_kv_heads).  A sequence with
 * seq_len <= 0 leaves its output rows untouched.
 *
 * The workspace is caller-owned scratch of at least GetWorkspaceSize bytes,
 * 256-byte aligned, contents undefined on entry.  Execute is asynchronous on
 * `stream` (NULL = the default stream), performs no allocation and no
 * host<->device synchronisation.
 */
#ifndef __INFINIOP_PAGED_ATTENTION_API_H__
#define __INFINIOP_PAGED_ATTENTION_API_H__

#include "../operator_descriptor.h"

typedef struct InfiniopDescriptor *infiniopPagedAttentionDescriptor_t;

/* reference include/infiniop/ops/paged_attention.h:33-43 */
__INFINI_C __export infiniStatus_t infiniopCreatePagedAttentionDescriptor(
    infiniopHandle_t handle,
    infiniopPagedAttentionDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    float scale);

/* reference include/infiniop/ops/paged_attention.h:52-53 */
__INFINI_C __export infiniStatus_t infiniopGetPagedAttentionWorkspaceSize(
    infiniopPagedAttentionDescriptor_t desc, size_t *size);

/* reference include/infiniop/ops/paged_attention.h:71-82 */
__INFINI_C __export infiniStatus_t infiniopPagedAttention(
    infiniopPagedAttentionDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    const void *k_cache,
    const void *v_cache,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    void *stream);

/*
 * No counterpart in the reference.  Same operation as infiniopPagedAttention, for callers that
 * cannot provide a workspace because they cannot allocate device memory (all of HBM already given
 * to the KV pool, a frozen allocator, a host framework that owns every buffer): the scratch is a
 * 32 MiB array inside this library (INFINIOP_PAGED_ATTENTION_STATIC_WORKSPACE_BYTES).  Descriptors
 * that need more are refused with INFINI_STATUS_INSUFFICIENT_WORKSPACE.  The first call on a device
 * resolves the array's address; under the CUDA runtime's lazy module loading that is also the moment
 * the device sets the 32 MiB aside, so make that call at start-up, while the memory is still free
 * (before the KV pool takes the rest) and before any stream capture; from then on the device holds
 * the array until the process exits and no call takes further memory.  All calls on a device share
 * the array: calls that overlap on the GPU race.  Calls no allocating routine.
 */
#define INFINIOP_PAGED_ATTENTION_STATIC_WORKSPACE_BYTES (32u << 20)
__INFINI_C __export infiniStatus_t infiniopPagedAttentionStaticWorkspace(
    infiniopPagedAttentionDescriptor_t desc,
    void *out,
    const void *q,
    const void *k_cache,
    const void *v_cache,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    void *stream);

/* reference include/infiniop/ops/paged_attention.h:90-91 */
__INFINI_C __export infiniStatus_t infiniopDestroyPagedAttentionDescriptor(
    infiniopPagedAttentionDescriptor_t desc);

/* No reference counterpart.  infiniopPagedAttention with every output row stored to `num_outs`
 * buffers (1..8) that all have the shape and strides of the descriptor's `out`; outs[0] is the
 * ordinary output.  The buffers may live on other GPUs whose memory this GPU can address (peer
 * access, symmetric memory): the KV-head-sharded mode hands in the address of its head slice
 * inside every rank's full output, and the all-gather that would follow the kernel is not needed -
 * only a barrier across the ranks before anyone reads its full output.  That one barrier does not
 * protect a buffer that is reused by the next step: a rank that passed it may start the next step and
 * store new rows into a peer's buffer while that peer still reads this step's.  Alternate between two
 * sets of buffers from step to step (then one barrier per step is enough), or synchronise the ranks a
 * second time between the reads and the next step's stores.  Sequences with seq_len <= 0 leave their
 * rows untouched in every buffer. */
__INFINI_C __export infiniStatus_t infiniopPagedAttentionMultiOut(
    infiniopPagedAttentionDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *const *outs,
    size_t num_outs,
    const void *q,
    const void *k_cache,
    const void *v_cache,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    void *stream);

#endif
