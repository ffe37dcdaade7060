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
 */
#ifndef __INFINIOP_PAGED_DECODE_STEP_API_H__
#define __INFINIOP_PAGED_DECODE_STEP_API_H__

#include "../operator_descriptor.h"

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

/* no reference counterpart; same size as infiniopGetPagedAttentionWorkspaceSize for the same problem */
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

/* no reference counterpart */
__INFINI_C __export infiniStatus_t infiniopDestroyPagedDecodeStepDescriptor(
    infiniopPagedDecodeStepDescriptor_t desc);

#endif
