/*
 * Rotary position embedding.  Replaces reference include/infiniop/ops/rope.h:6-40 with identical
 * signatures and enum values.
 *
 * Tensors:
 *   y, x       [seqlen, nhead, dhead] or [batch, seqlen, nhead, dhead]   F16 | BF16 | F32 | F64, the same
 *              shape, last stride 1, any other strides; y may alias x (in place)
 *   pos_ids    [seqlen] (shared by the batch) or [batch, seqlen], dense, any integer type
 *   sin_table  [table_len, dhead / 2]   contiguous, dtype of x
 *   cos_table  [table_len, dhead / 2]   contiguous, dtype of x
 *
 * For every (batch, token, head) row and i in [0, dhead / 2), with s = sin_table[pos][i],
 * c = cos_table[pos][i] and (a, b) the pair of the algorithm:
 *   GPT_J     a = 2 i,  b = 2 i + 1      (interleaved pairs)
 *   GPT_NEOX  a = i,    b = i + dhead/2  (first half against second half)
 *   y[a] = x[a] c - x[b] s,   y[b] = x[a] s + x[b] c
 * Arithmetic (reference src/infiniop/ops/rope/cpu/rope_cpu.cc:78-101): F16 / BF16 operands are
 * widened to fp32, each product and the sum are rounded separately (no fused multiply-add) and the
 * result is rounded once, to nearest even, to the tensor's type; F32 and F64 compute in their own
 * type.  A position outside [0, table_len) leaves its rows as plain copies of x (the reference
 * reads outside the tables there).  Workspace size is 0.
 */
#ifndef __INFINIOP_ROPE_API_H__
#define __INFINIOP_ROPE_API_H__

#include "../operator_descriptor.h"

/* reference include/infiniop/ops/rope.h:6-12 */
typedef enum {
    INFINIOP_ROPE_ALGO_GPT_J = 0,
    INFINIOP_ROPE_ALGO_GPT_NEOX = 1,
    INFINIOP_ROPE_ALGO_COUNT = 2,
} infiniopRoPEAlgo_t;

typedef struct InfiniopDescriptor *infiniopRoPEDescriptor_t;

/* reference include/infiniop/ops/rope.h:16-24 */
__INFINI_C __export infiniStatus_t infiniopCreateRoPEDescriptor(
    infiniopHandle_t handle,
    infiniopRoPEDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t y,
    infiniopTensorDescriptor_t x,
    infiniopTensorDescriptor_t pos_ids,
    infiniopTensorDescriptor_t sin_table,
    infiniopTensorDescriptor_t cos_table,
    infiniopRoPEAlgo_t algo);

/* reference include/infiniop/ops/rope.h:26 */
__INFINI_C __export infiniStatus_t infiniopGetRoPEWorkspaceSize(infiniopRoPEDescriptor_t desc, size_t *size);

/* reference include/infiniop/ops/rope.h:28-37 */
__INFINI_C __export infiniStatus_t infiniopRoPE(
    infiniopRoPEDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *y,
    const void *x,
    void const *pos_ids,
    void const *sin_table,
    void const *cos_table,
    void *stream);

/* reference include/infiniop/ops/rope.h:39 */
__INFINI_C __export infiniStatus_t infiniopDestroyRoPEDescriptor(infiniopRoPEDescriptor_t desc);

#endif
