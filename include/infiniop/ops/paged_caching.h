/*
 * Paged caching: scatter new K/V rows into the paged cache pools.  Replaces
 * reference include/infiniop/ops/paged_caching.h:24-75 with identical signatures.
 *
 * Tensors:
 *   k_cache       [num_blocks, num_kv_heads, block_size, head_size]   F16 | BF16 | F32
 *   v_cache       [num_blocks, num_kv_heads, block_size, v_head_size] (any block/head/slot strides)
 *   k             [num_tokens, num_kv_heads, head_size]
 *   v             [num_tokens, num_kv_heads, v_head_size]
 *   slot_mapping  [num_tokens] I64
 *
 * Row i goes to cache[slot / block_size, :, slot % block_size, :] with
 * slot = slot_mapping[i]; a negative slot marks padding and is skipped.  The copy
 * is bit-exact.  Workspace size is 0.
 */
#ifndef __INFINIOP_PAGED_CACHING_API_H__
#define __INFINIOP_PAGED_CACHING_API_H__

#include "../operator_descriptor.h"

typedef struct InfiniopDescriptor *infiniopPagedCachingDescriptor_t;

/* reference include/infiniop/ops/paged_caching.h:24-31 */
__INFINI_C __export infiniStatus_t infiniopCreatePagedCachingDescriptor(
    infiniopHandle_t handle,
    infiniopPagedCachingDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t k_desc,
    infiniopTensorDescriptor_t v_desc,
    infiniopTensorDescriptor_t slot_mapping_desc);

/* reference include/infiniop/ops/paged_caching.h:40-41 */
__INFINI_C __export infiniStatus_t infiniopGetPagedCachingWorkspaceSize(
    infiniopPagedCachingDescriptor_t desc, size_t *size);

/* reference include/infiniop/ops/paged_caching.h:57-66 */
__INFINI_C __export infiniStatus_t infiniopPagedCaching(
    infiniopPagedCachingDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *k_cache,
    void *v_cache,
    const void *k,
    const void *v,
    const void *slot_mapping,
    void *stream);

/* reference include/infiniop/ops/paged_caching.h:74-75 */
__INFINI_C __export infiniStatus_t infiniopDestroyPagedCachingDescriptor(
    infiniopPagedCachingDescriptor_t desc);

#endif
