/* InfiniCCL: collectives over the devices InfiniRT manages.
 *
 * Declares what the reference declares in include/infiniccl.h:6-114, for the NVIDIA device type
 * only; every entry point forwards to NCCL (reference src/infiniccl/cuda/infiniccl_cuda.cu).
 * A communicator belongs to one device; calls are asynchronous on the given stream (NULL = the
 * default stream) and return INFINI_STATUS_INTERNAL_ERROR when NCCL reports a failure.
 *
 * On this path the library is used by the KV-head-sharded decode mode to put the per-rank
 * [seqs, heads / N, head_size] outputs together (infinicclAllGather); the sequence-sharded mode
 * needs no collective at all.
 */
#ifndef __INFINICCL_API_H__
#define __INFINICCL_API_H__

#include "infinirt.h"

/* reference include/infiniccl.h:6-12 */
typedef enum {
    INFINICCL_SUM = 0,
    INFINICCL_PROD = 1,
    INFINICCL_MAX = 2,
    INFINICCL_MIN = 3,
    INFINICCL_AVG = 4,
} infinicclReduceOp_t;

struct InfinicclComm;
typedef struct InfinicclComm *infinicclComm_t;

/* Opaque rendezvous token: made on one rank, carried to the others by the caller
 * (reference include/infiniccl.h:18-22). */
#define INFINICCL_UNIQUE_ID_BYTES 128
typedef struct {
    char internal[INFINICCL_UNIQUE_ID_BYTES];
} infinicclUniqueId_t;

/* One process, several devices: comms[i] is rank i on device_ids[i] (reference :24-28). */
__INFINI_C __export infiniStatus_t infinicclCommInitAll(infiniDevice_t device_type, infinicclComm_t *comms, int ndevice,
                                                        const int *device_ids);
/* One process per device: rank 0 makes the token, every rank joins with it on its current
 * device (reference :30-37). */
__INFINI_C __export infiniStatus_t infinicclGetUniqueId(infinicclUniqueId_t *unique_id);
__INFINI_C __export infiniStatus_t infinicclCommInitRank(infinicclComm_t *comm, int nranks, infinicclUniqueId_t comm_id, int rank);
/* NULL is accepted and does nothing (reference src/infiniccl/infiniccl.cc:98-101). */
__INFINI_C __export infiniStatus_t infinicclCommDestroy(infinicclComm_t comm);

/* Brackets calls that must be issued together (one thread driving several communicators,
 * or matched send/recv pairs); reference :41-43. */
__INFINI_C __export infiniStatus_t infinicclGroupStart(infinicclComm_t comm);
__INFINI_C __export infiniStatus_t infinicclGroupEnd(infinicclComm_t comm);

/* Element types: F32, F16, BF16, I32, I64, U32, U64; anything else is
 * INFINI_STATUS_BAD_TENSOR_DTYPE.  Counts are in elements.  Reference :45-114. */
__INFINI_C __export infiniStatus_t infinicclAllReduce(void *sendbuf, void *recvbuf, size_t count, infiniDtype_t dataype,
                                                      infinicclReduceOp_t op, infinicclComm_t comm, infinirtStream_t stream);
__INFINI_C __export infiniStatus_t infinicclBroadcast(const void *sendbuf, void *recvbuf, size_t count, infiniDtype_t datatype,
                                                      int root, infinicclComm_t comm, infinirtStream_t stream);
__INFINI_C __export infiniStatus_t infinicclSend(const void *sendbuf, size_t count, infiniDtype_t datatype, int peer,
                                                 infinicclComm_t comm, infinirtStream_t stream);
__INFINI_C __export infiniStatus_t infinicclRecv(void *recvbuf, size_t count, infiniDtype_t datatype, int peer,
                                                 infinicclComm_t comm, infinirtStream_t stream);
/* recvbuf holds world_size * send_count elements, rank-major. */
__INFINI_C __export infiniStatus_t infinicclAllGather(void *sendbuf, void *recvbuf, size_t send_count, infiniDtype_t dataype,
                                                      infinicclComm_t comm, infinirtStream_t stream);
/* Rank r contributes recv_counts[r] elements; recvbuf is their concatenation in rank order. */
__INFINI_C __export infiniStatus_t infinicclAllGatherV(void *sendbuf, void *recvbuf, const size_t *recv_counts, int nranks,
                                                       infiniDtype_t dataype, infinicclComm_t comm, infinirtStream_t stream);
/* sendbuf holds world_size * recv_count elements; rank r receives the reduction of slice r. */
__INFINI_C __export infiniStatus_t infinicclReduceScatter(void *sendbuf, void *recvbuf, size_t recv_count, infiniDtype_t dataype,
                                                          infinicclReduceOp_t op, infinicclComm_t comm, infinirtStream_t stream);
/* Slice r of sendbuf has send_counts[r] elements. */
__INFINI_C __export infiniStatus_t infinicclReduceScatterV(void *sendbuf, void *recvbuf, const size_t *send_counts, int nranks,
                                                           infiniDtype_t dataype, infinicclReduceOp_t op, infinicclComm_t comm,
                                                           infinirtStream_t stream);

#endif /* __INFINICCL_API_H__ */
