/*
 * Library context handle.  Replaces reference include/infiniop/handle.h:10-12.
 *
 * infiniopCreateHandle binds the new handle to the calling thread's current
 * infinirt device (reference src/infiniop/devices/handle.cc:26-34).  The object
 * behind the pointer begins with {int device; int device_id;} - callers read
 * those two ints (reference src/infiniop/handle.h:6-9).  Only INFINI_DEVICE_NVIDIA
 * on an sm_100 GPU is accepted; anything else returns
 * INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED / ..._ARCHITECTURE_NOT_SUPPORTED.
 */
#ifndef __INFINIOP_HANDLE_API_H__
#define __INFINIOP_HANDLE_API_H__

#include "../infinicore.h"

struct InfiniopHandle;
typedef struct InfiniopHandle *infiniopHandle_t;

__INFINI_C __export infiniStatus_t infiniopCreateHandle(infiniopHandle_t *handle_ptr);
__INFINI_C __export infiniStatus_t infiniopDestroyHandle(infiniopHandle_t handle);

#endif
