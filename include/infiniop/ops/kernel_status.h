/*
 * Status the kernels of this library leave behind.  No counterpart in the reference, whose kernels
 * have nothing to report: they never wait on anything and never check an index
 * (reference src/infiniop/ops/paged_caching/cuda/kernel.cuh:60-78 stores to whatever slot it is given).
 *
 * Here two things can go wrong inside a launch without the launch itself failing:
 *   - a worker's bounded wait for one of its own TMA copies runs out (about 2 s; the copy engine never
 *     delivered).  The worker gives up, lets its other copies land and returns; the rows it was
 *     responsible for are missing from the output;
 *   - with index checking switched on (INFINIOP_PAGED_CHECK_INDICES=1 when the descriptor is created),
 *     a block-table entry or a cache slot lies outside the pool.  The kernel reads block 0 instead /
 *     skips the row, where the unchecked kernels - like the reference's - would touch foreign memory.
 * Each device keeps one sticky word of flags for all of this library's kernels.
 */
#ifndef __INFINIOP_KERNEL_STATUS_API_H__
#define __INFINIOP_KERNEL_STATUS_API_H__

#include "../handle.h"

#define INFINIOP_KERNEL_FLAG_WAIT_EXPIRED 1u        /* a bounded wait for a TMA copy or an MMA ran out */
#define INFINIOP_KERNEL_FLAG_BLOCK_OUT_OF_RANGE 2u  /* a block-table entry was < 0 or >= num_blocks (checked mode) */
#define INFINIOP_KERNEL_FLAG_SLOT_OUT_OF_RANGE 4u   /* a slot was >= num_blocks * block_size (checked mode) */

/*
 * Waits for `stream` (NULL: the default stream) on the handle's device, returns the device's flag
 * word in *flags and clears it.  0 means every kernel this library ran on the device since the last
 * call did all of its work.  Call it with that device current.  Flags raised by kernels still running
 * on OTHER streams while this call executes may be lost between its read and its clear.
 */
__INFINI_C __export infiniStatus_t infiniopGetKernelStatus(infiniopHandle_t handle, void *stream, unsigned int *flags);

#endif
