/* Umbrella header for the operator library (the subset this library implements:
 * handle, tensor/operator descriptors, paged_attention, paged_attention_prefill, paged_caching, paged_decode_step, rope, kv_caching, kernel_status). */
#ifndef __INFINIOP_API_H__
#define __INFINIOP_API_H__

#include "infiniop/handle.h"
#include "infiniop/operator_descriptor.h"
#include "infiniop/ops/kernel_status.h"
#include "infiniop/ops/kv_caching.h"
#include "infiniop/ops/paged_attention.h"
#include "infiniop/ops/paged_attention_prefill.h"
#include "infiniop/ops/paged_caching.h"
#include "infiniop/ops/paged_decode_step.h"
#include "infiniop/ops/rope.h"
#include "infiniop/tensor_descriptor.h"

#endif
