/*
 * Paged-attention prefill: a chunk of new query tokens per sequence (packed, variable length)
 * attends causally to that sequence's paged KV cache, which already contains the new tokens' K/V.
 * Replaces reference include/infiniop/ops/paged_attention_prefill.h:33-100 with identical signatures.
 *
 * Tensors:
 *   out             [total_q_tokens, num_heads, value_size]      F16 | BF16
 *   q               [total_q_tokens, num_heads, head_size]       same dtype (packed over sequences)
 *   k_cache/v_cache [num_blocks, num_kv_heads, block_size, head_size | value_size]
 *   block_tables    [num_seqs, max_num_blocks_per_seq]           I64 | I32 | U32
 *   seq_lens        [num_seqs]      total KV length of each sequence INCLUDING its new tokens
 *   cum_seq_lens_q  [num_seqs + 1]  prefix sum of the new-token counts (same index dtype)
 *   alibi_slopes    [num_heads] F32, optional
 *
 * New token t (0-based within its chunk of n) of sequence i sits at KV position
 * seq_lens[i] - n + t and attends positions 0 .. seq_lens[i] - n + t
 * (reference test/infiniop/paged_attention_prefill.py:96-140).
 */
#ifndef __INFINIOP_PAGED_ATTENTION_PREFILL_API_H__
#define __INFINIOP_PAGED_ATTENTION_PREFILL_API_H__

#include "../operator_descriptor.h"

typedef struct InfiniopDescriptor *infiniopPagedAttentionPrefillDescriptor_t;

/* reference include/infiniop/ops/paged_attention_prefill.h:33-44 */
__INFINI_C __export infiniStatus_t infiniopCreatePagedAttentionPrefillDescriptor(
    infiniopHandle_t handle,
    infiniopPagedAttentionPrefillDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t cum_seq_lens_q_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    float scale);

/* reference include/infiniop/ops/paged_attention_prefill.h:49-50 */
__INFINI_C __export infiniStatus_t infiniopGetPagedAttentionPrefillWorkspaceSize(
    infiniopPagedAttentionPrefillDescriptor_t desc, size_t *size);

/* reference include/infiniop/ops/paged_attention_prefill.h:68-80 */
__INFINI_C __export infiniStatus_t infiniopPagedAttentionPrefill(
    infiniopPagedAttentionPrefillDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    const void *k_cache,
    const void *v_cache,
    const void *block_tables,
    const void *seq_lens,
    const void *cum_seq_lens_q,
    const void *alibi_slopes,
    void *stream);

/* reference include/infiniop/ops/paged_attention_prefill.h:85-86 */
__INFINI_C __export infiniStatus_t infiniopDestroyPagedAttentionPrefillDescriptor(
    infiniopPagedAttentionPrefillDescriptor_t desc);

#endif
