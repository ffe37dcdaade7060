/*
 * Paged decode step: append each sequence's newest K/V row to the paged cache and attend over the
 * sequence, as one operator.  No counterpart in the reference: there a decode layer calls
 * infiniopPagedCaching (include/infiniop/ops/paged_caching.h:57-66) and then infiniopPagedAttention
 * (include/infiniop/ops/paged_attention.h:66-77); this entry point does the work of that pair in
 * one attention launch (plus its small combine launch), so one kernel launch per layer goes away.
 *
 * Tensors (dtypes, strides and status codes as for infiniopPagedAttention):
 *   out           [num_seqs, num_heads, head_size]
 *   q             [num_seqs, num_heads, head_size]
 *   k_cache       [num_blocks, num_kv_heads, block_size, head_size]   read AND written
 *   v_cache       [num_blocks, num_kv_heads, block_size, head_size]   read AND written
 *   new_k, new_v  [num_seqs, num_kv_heads, head_size]   last stride 1, dense heads (stride(1) == head_size)
 *   block_tables  [num_seqs, max_blocks_per_seq], seq_lens [num_seqs]   I64 | I32 | U32, the same type
 *   alibi_slopes  [num_heads] F32, optional
 *
 * For every sequence i with seq_lens[i] >= 1 (the length INCLUDING the new token):
 *   position n = seq_lens[i] - 1 lives at slot (block_tables[i][n / block_size], n % block_size);
 *   k_cache[that slot] = new_k[i], v_cache[that slot] = new_v[i]   (bit-exact copies), then
 *   out[i] = attention of q[i] over positions 0..n of sequence i.
 * Sequences with seq_lens[i] <= 0 are left alone (no append, output row untouched).  The result
 * equals infiniopPagedCaching with slot_mapping[i] = block * block_size + n % block_size followed
 * by infiniopPagedAttention, cache contents included.
 *
 * RoPE form (infiniopCreatePagedDecodeStepRoPEDescriptor / infiniopPagedDecodeStepRoPE): additionally
 * does the work of the two infiniopRoPE calls (include/infiniop/ops/rope.h) a decode layer issues
 * before caching - on q and on new_k, each viewed as [num_seqs, heads, head_size] with
 *   pos_ids    [num_seqs]                    any integer type, dense
 *   sin_table  [table_len, head_size / 2]    contiguous, dtype of q
 *   cos_table  [table_len, head_size / 2]    contiguous, dtype of q
 * The cache receives the ROTATED K row and the attention uses the rotated q; q and new_k themselves
 * are not modified (the rotated rows live in the workspace).  Results equal infiniopRoPE(q),
 * infiniopRoPE(new_k), infiniopPagedCaching, infiniopPagedAttention in that order; the rotation is
 * bit-exact with infiniopRoPE.  The workspace must be 256-byte aligned.
 */
#ifndef __INFINIOP_PAGED_DECODE_STEP_API_H__
#define __INFINIOP_PAGED_DECODE_STEP_API_H__

#include "../operator_descriptor.h"
#include "rope.h"

typedef struct InfiniopDescriptor *infiniopPagedDecodeStepDescriptor_t;

/* no reference counterpart (see above) */
__INFINI_C __export infiniStatus_t infiniopCreatePagedDecodeStepDescriptor(
    infiniopHandle_t handle,
    infiniopPagedDecodeStepDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t new_k_desc,
    infiniopTensorDescriptor_t new_v_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    float scale);

/* no reference counterpart: infiniopCreatePagedDecodeStepDescriptor plus the position ids and tables of
 * infiniopCreateRoPEDescriptor (reference include/infiniop/ops/rope.h:16-24) */
__INFINI_C __export infiniStatus_t infiniopCreatePagedDecodeStepRoPEDescriptor(
    infiniopHandle_t handle,
    infiniopPagedDecodeStepDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t new_k_desc,
    infiniopTensorDescriptor_t new_v_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    infiniopTensorDescriptor_t pos_ids_desc,
    infiniopTensorDescriptor_t sin_table_desc,
    infiniopTensorDescriptor_t cos_table_desc,
    infiniopRoPEAlgo_t algo,
    float scale);

/* no reference counterpart; the size infiniopGetPagedAttentionWorkspaceSize reports for the same problem
 * (the RoPE form adds room for the rotated q and K rows) */
__INFINI_C __export infiniStatus_t infiniopGetPagedDecodeStepWorkspaceSize(
    infiniopPagedDecodeStepDescriptor_t desc, size_t *size);

/* no reference counterpart */
__INFINI_C __export infiniStatus_t infiniopPagedDecodeStep(
    infiniopPagedDecodeStepDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    void *k_cache,
    void *v_cache,
    const void *new_k,
    const void *new_v,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    void *stream);

/* no reference counterpart; for descriptors of infiniopCreatePagedDecodeStepRoPEDescriptor only */
__INFINI_C __export infiniStatus_t infiniopPagedDecodeStepRoPE(
    infiniopPagedDecodeStepDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    void *k_cache,
    void *v_cache,
    const void *new_k,
    const void *new_v,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    const void *pos_ids,
    const void *sin_table,
    const void *cos_table,
    void *stream);

/* no reference counterpart */
__INFINI_C __export infiniStatus_t infiniopDestroyPagedDecodeStepDescriptor(
    infiniopPagedDecodeStepDescriptor_t desc);

#endif
