/*
 * Tensor descriptor: dtype + shape + element strides.  Replaces reference
 * include/infiniop/tensor_descriptor.h:10-12; semantics follow reference
 * src/infiniop/tensor_descriptor.cc:8-29 (strides == NULL means row-major
 * contiguous).  The descriptor is opaque to callers and may be destroyed as soon
 * as the operator descriptor that consumed it has been created.
 */
#ifndef __INFINIOP_TENSOR_DESCRIPTOR_API_H__
#define __INFINIOP_TENSOR_DESCRIPTOR_API_H__

#include "../infinicore.h"

struct InfiniopTensorDescriptor;
typedef struct InfiniopTensorDescriptor *infiniopTensorDescriptor_t;

__INFINI_C __export infiniStatus_t infiniopCreateTensorDescriptor(
    infiniopTensorDescriptor_t *desc_ptr,
    size_t ndim,
    const size_t *shape,
    const ptrdiff_t *strides,
    infiniDtype_t dtype);

__INFINI_C __export infiniStatus_t infiniopDestroyTensorDescriptor(infiniopTensorDescriptor_t desc);

#endif
