/*
 * Contiguous (non-paged) KV cache update: append `seq_len` new rows per sequence behind the rows a
 * sequence already holds.  Replaces reference include/infiniop/ops/kv_caching.h:6-32 with identical
 * signatures.  It is the non-paged sibling of infiniopPagedCaching in the reference's decode layers.
 *
 * Tensors (any strides, the last one included):
 *   k_cache, v_cache   [batch, num_kv_heads, max_seq_len, hidden]   F16 | BF16 | F32, the same shape
 *   k, v               [batch, num_kv_heads, seq_len, hidden]       dtype of the caches, the same shape
 *   past_kv_lengths    [batch]   I32 | I64, dense
 *
 *   k_cache[b, h, past_kv_lengths[b] + s, :] = k[b, h, s, :]   (v likewise), bit-exact copies.
 *
 * Rows whose destination falls outside [0, max_seq_len) are skipped (the reference writes outside the
 * cache there).  batch, num_kv_heads and hidden of k / v must equal the caches' (the reference accepts a
 * match in any one of the three, src/infiniop/ops/kv_caching/info.h:57-60, and then indexes out of
 * bounds).  Workspace size is 0.
 */
#ifndef __INFINIOP_KV_CACHING_API_H__
#define __INFINIOP_KV_CACHING_API_H__

#include "../operator_descriptor.h"

typedef struct InfiniopDescriptor *infiniopKVCachingDescriptor_t;

/* reference include/infiniop/ops/kv_caching.h:8-15 */
__INFINI_C __export infiniStatus_t infiniopCreateKVCachingDescriptor(
    infiniopHandle_t handle,
    infiniopKVCachingDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t k_cache,
    infiniopTensorDescriptor_t v_cache,
    infiniopTensorDescriptor_t k,
    infiniopTensorDescriptor_t v,
    infiniopTensorDescriptor_t past_kv_lengths);

/* reference include/infiniop/ops/kv_caching.h:17 */
__INFINI_C __export infiniStatus_t infiniopGetKVCachingWorkspaceSize(infiniopKVCachingDescriptor_t desc, size_t *size);

/* reference include/infiniop/ops/kv_caching.h:19-27 */
__INFINI_C __export infiniStatus_t infiniopKVCaching(
    infiniopKVCachingDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *k_cache,
    void *v_cache,
    const void *k,
    const void *v,
    const void *past_kv_lengths,
    void *stream);

/* reference include/infiniop/ops/kv_caching.h:29 */
__INFINI_C __export infiniStatus_t infiniopDestroyKVCachingDescriptor(infiniopKVCachingDescriptor_t desc);

#endif
