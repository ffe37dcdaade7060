/*
 * Base of every operator descriptor.  Replaces reference
 * include/infiniop/operator_descriptor.h:7-11.  The object behind the pointer
 * begins with {int device_type; int device_id;} (reference
 * src/infiniop/operator.h:6-9), which ctypes callers read directly.
 */
#ifndef __INFINIOP_OPERATOR_DESCRIPTOR_API_H__
#define __INFINIOP_OPERATOR_DESCRIPTOR_API_H__

#include "handle.h"
#include "tensor_descriptor.h"

struct InfiniopDescriptor;

__INFINI_C __export infiniStatus_t infiniopGetDescriptorDeviceType(
    const struct InfiniopDescriptor *desc_ptr, infiniDevice_t *device_type);
__INFINI_C __export infiniStatus_t infiniopGetDescriptorDeviceId(
    const struct InfiniopDescriptor *desc_ptr, int *device_id);

#endif
