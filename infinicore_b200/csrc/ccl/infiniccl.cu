// libinfiniccl: the InfiniCCL C ABI over NCCL for B200 (NVLink 5 / NVSwitch underneath).
//
// Behaviour follows the reference's dispatcher and CUDA backend (src/infiniccl/infiniccl.cc,
// src/infiniccl/cuda/infiniccl_cuda.cu): same argument checks and status codes, the variable-count
// collectives expressed as one NCCL group of per-root broadcasts / reductions.  Unlike the reference,
// an element type or reduction outside the supported set is refused with a status code instead of
// aborting the process.
#include "infiniccl.h"
#include "infinirt.h"

#include <cstdio>
#include <cstring>
#include <cuda_runtime.h>
#include <nccl.h>
#include <vector>

struct InfinicclComm {
    infiniDevice_t device_type;
    int device_id; // the CUDA device, not the rank
    ncclComm_t comm;
    int rank;
    int world_size;
};

static_assert(sizeof(ncclUniqueId) <= INFINICCL_UNIQUE_ID_BYTES, "rendezvous token must hold an NCCL id");

namespace {

bool toNccl(infiniDtype_t t, ncclDataType_t *out, size_t *bytes) {
    switch (t) {
    case INFINI_DTYPE_I32:
        *out = ncclInt32, *bytes = 4;
        return true;
    case INFINI_DTYPE_I64:
        *out = ncclInt64, *bytes = 8;
        return true;
    case INFINI_DTYPE_U32:
        *out = ncclUint32, *bytes = 4;
        return true;
    case INFINI_DTYPE_U64:
        *out = ncclUint64, *bytes = 8;
        return true;
    case INFINI_DTYPE_F32:
        *out = ncclFloat, *bytes = 4;
        return true;
    case INFINI_DTYPE_F16:
        *out = ncclHalf, *bytes = 2;
        return true;
    case INFINI_DTYPE_BF16:
        *out = ncclBfloat16, *bytes = 2;
        return true;
    default:
        return false;
    }
}

bool toNccl(infinicclReduceOp_t op, ncclRedOp_t *out) {
    switch (op) {
    case INFINICCL_SUM:
        *out = ncclSum;
        return true;
    case INFINICCL_PROD:
        *out = ncclProd;
        return true;
    case INFINICCL_MAX:
        *out = ncclMax;
        return true;
    case INFINICCL_MIN:
        *out = ncclMin;
        return true;
    case INFINICCL_AVG:
        *out = ncclAvg;
        return true;
    default:
        return false;
    }
}

infiniStatus_t fromNccl(ncclResult_t r, const char *what) {
    if (r == ncclSuccess) {
        return INFINI_STATUS_SUCCESS;
    }
    std::fprintf(stderr, "[infiniccl] %s: %s\n", what, ncclGetErrorString(r));
    return INFINI_STATUS_INTERNAL_ERROR;
}

cudaStream_t cudaStreamOf(infinirtStream_t s) { return static_cast<cudaStream_t>(s); }

// Brackets one collective (or one whole group of them) with the event pair that libinfinirt turns into the
// resource snapshot's communication figures (reference src/infiniccl/cuda/infiniccl_cuda.cu records the same
// samples).  Inside a caller's infinicclGroupStart / GroupEnd the launches only happen at GroupEnd, so the
// calls in between just add their payload and the group is bracketed as one sample.
thread_local int t_group_depth = 0;
thread_local uint64_t t_group_bytes = 0;
thread_local infinirtStream_t t_group_stream = nullptr;

class Sampled {
public:
    Sampled(infinirtStream_t stream, uint64_t bytes) : stream_(stream), bytes_(bytes) {
        if (t_group_depth > 0) {
            t_group_bytes += bytes;
            t_group_stream = stream;
        } else {
            (void)infinirtCommunicationBegin(stream, &sample_);
        }
    }
    ~Sampled() {
        if (sample_ != nullptr) {
            (void)infinirtCommunicationEnd(sample_, stream_, launched_ ? bytes_ : 0);
        }
    }
    void launched() { launched_ = true; }
    Sampled(const Sampled &) = delete;
    Sampled &operator=(const Sampled &) = delete;

private:
    infinirtStream_t stream_;
    uint64_t bytes_;
    void *sample_ = nullptr;
    bool launched_ = false;
};

bool nvidiaFamily(infiniDevice_t d) { return d == INFINI_DEVICE_NVIDIA; }

} // namespace

#define CCL_NCCL(call)                                        \
    do {                                                      \
        const infiniStatus_t st__ = fromNccl((call), #call);  \
        if (st__ != INFINI_STATUS_SUCCESS) {                  \
            return st__;                                      \
        }                                                     \
    } while (0)

#define CCL_REQUIRE(cond, status) \
    do {                          \
        if (!(cond)) {            \
            return (status);      \
        }                         \
    } while (0)

__INFINI_C infiniStatus_t infinicclCommInitAll(infiniDevice_t device_type, infinicclComm_t *comms, int ndevice, const int *device_ids) {
    CCL_REQUIRE(nvidiaFamily(device_type), INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);
    CCL_REQUIRE(comms != nullptr && device_ids != nullptr, INFINI_STATUS_NULL_POINTER);
    CCL_REQUIRE(ndevice > 0, INFINI_STATUS_BAD_PARAM);
    std::vector<ncclComm_t> raw(ndevice);
    CCL_NCCL(ncclCommInitAll(raw.data(), ndevice, device_ids));
    for (int i = 0; i < ndevice; ++i) {
        comms[i] = new InfinicclComm{INFINI_DEVICE_NVIDIA, device_ids[i], raw[i], i, ndevice};
    }
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclGetUniqueId(infinicclUniqueId_t *unique_id) {
    CCL_REQUIRE(unique_id != nullptr, INFINI_STATUS_NULL_POINTER);
    infiniDevice_t device_type;
    const infiniStatus_t st = infinirtGetDevice(&device_type, nullptr);
    CCL_REQUIRE(st == INFINI_STATUS_SUCCESS, st);
    CCL_REQUIRE(nvidiaFamily(device_type), INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);
    ncclUniqueId id;
    CCL_NCCL(ncclGetUniqueId(&id));
    std::memset(unique_id, 0, sizeof(*unique_id));
    std::memcpy(unique_id, &id, sizeof(id));
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclCommInitRank(infinicclComm_t *comm, int nranks, infinicclUniqueId_t comm_id, int rank) {
    CCL_REQUIRE(comm != nullptr, INFINI_STATUS_NULL_POINTER);
    infiniDevice_t device_type;
    int device_id = 0;
    const infiniStatus_t st = infinirtGetDevice(&device_type, &device_id);
    CCL_REQUIRE(st == INFINI_STATUS_SUCCESS, st);
    CCL_REQUIRE(nvidiaFamily(device_type), INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);
    CCL_REQUIRE(nranks > 0 && rank >= 0 && rank < nranks, INFINI_STATUS_BAD_PARAM);
    ncclUniqueId id;
    std::memcpy(&id, &comm_id, sizeof(id));
    ncclComm_t raw;
    CCL_NCCL(ncclCommInitRank(&raw, nranks, id, rank));
    *comm = new InfinicclComm{device_type, device_id, raw, rank, nranks};
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclCommDestroy(infinicclComm_t comm) {
    if (comm == nullptr) {
        return INFINI_STATUS_SUCCESS;
    }
    const infiniStatus_t st = fromNccl(ncclCommDestroy(comm->comm), "ncclCommDestroy");
    delete comm;
    return st;
}

__INFINI_C infiniStatus_t infinicclGroupStart(infinicclComm_t comm) {
    CCL_REQUIRE(comm != nullptr, INFINI_STATUS_NULL_POINTER);
    CCL_NCCL(ncclGroupStart());
    if (t_group_depth++ == 0) {
        t_group_bytes = 0;
    }
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclGroupEnd(infinicclComm_t comm) {
    CCL_REQUIRE(comm != nullptr, INFINI_STATUS_NULL_POINTER);
    if (t_group_depth > 0 && --t_group_depth == 0 && t_group_bytes > 0) {
        // the outermost group ends: everything queued since GroupStart is launched by this call
        void *sample = nullptr;
        (void)infinirtCommunicationBegin(t_group_stream, &sample);
        const ncclResult_t r = ncclGroupEnd();
        (void)infinirtCommunicationEnd(sample, t_group_stream, r == ncclSuccess ? t_group_bytes : 0);
        t_group_bytes = 0;
        return fromNccl(r, "ncclGroupEnd");
    }
    CCL_NCCL(ncclGroupEnd());
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclAllReduce(void *sendbuf, void *recvbuf, size_t count, infiniDtype_t datatype, infinicclReduceOp_t op,
                                             infinicclComm_t comm, infinirtStream_t stream) {
    CCL_REQUIRE(comm != nullptr, INFINI_STATUS_NULL_POINTER);
    ncclDataType_t dt;
    size_t esize;
    ncclRedOp_t rop;
    CCL_REQUIRE(toNccl(datatype, &dt, &esize), INFINI_STATUS_BAD_TENSOR_DTYPE);
    CCL_REQUIRE(toNccl(op, &rop), INFINI_STATUS_BAD_PARAM);
    Sampled sample(stream, count * esize);
    CCL_NCCL(ncclAllReduce(sendbuf, recvbuf, count, dt, rop, comm->comm, cudaStreamOf(stream)));
    sample.launched();
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclBroadcast(const void *sendbuf, void *recvbuf, size_t count, infiniDtype_t datatype, int root,
                                             infinicclComm_t comm, infinirtStream_t stream) {
    CCL_REQUIRE(sendbuf != nullptr && recvbuf != nullptr && comm != nullptr, INFINI_STATUS_NULL_POINTER);
    CCL_REQUIRE(root >= 0 && root < comm->world_size && count > 0, INFINI_STATUS_BAD_PARAM);
    ncclDataType_t dt;
    size_t esize;
    CCL_REQUIRE(toNccl(datatype, &dt, &esize), INFINI_STATUS_BAD_TENSOR_DTYPE);
    Sampled sample(stream, count * esize);
    CCL_NCCL(ncclBroadcast(sendbuf, recvbuf, count, dt, root, comm->comm, cudaStreamOf(stream)));
    sample.launched();
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclSend(const void *sendbuf, size_t count, infiniDtype_t datatype, int peer, infinicclComm_t comm,
                                        infinirtStream_t stream) {
    CCL_REQUIRE(sendbuf != nullptr && comm != nullptr, INFINI_STATUS_NULL_POINTER);
    CCL_REQUIRE(peer >= 0 && peer < comm->world_size && count > 0, INFINI_STATUS_BAD_PARAM);
    ncclDataType_t dt;
    size_t esize;
    CCL_REQUIRE(toNccl(datatype, &dt, &esize), INFINI_STATUS_BAD_TENSOR_DTYPE);
    Sampled sample(stream, count * esize);
    CCL_NCCL(ncclSend(sendbuf, count, dt, peer, comm->comm, cudaStreamOf(stream)));
    sample.launched();
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclRecv(void *recvbuf, size_t count, infiniDtype_t datatype, int peer, infinicclComm_t comm,
                                        infinirtStream_t stream) {
    CCL_REQUIRE(recvbuf != nullptr && comm != nullptr, INFINI_STATUS_NULL_POINTER);
    CCL_REQUIRE(peer >= 0 && peer < comm->world_size && count > 0, INFINI_STATUS_BAD_PARAM);
    ncclDataType_t dt;
    size_t esize;
    CCL_REQUIRE(toNccl(datatype, &dt, &esize), INFINI_STATUS_BAD_TENSOR_DTYPE);
    Sampled sample(stream, count * esize);
    CCL_NCCL(ncclRecv(recvbuf, count, dt, peer, comm->comm, cudaStreamOf(stream)));
    sample.launched();
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclAllGather(void *sendbuf, void *recvbuf, size_t send_count, infiniDtype_t datatype, infinicclComm_t comm,
                                             infinirtStream_t stream) {
    CCL_REQUIRE(comm != nullptr, INFINI_STATUS_NULL_POINTER);
    ncclDataType_t dt;
    size_t esize;
    CCL_REQUIRE(toNccl(datatype, &dt, &esize), INFINI_STATUS_BAD_TENSOR_DTYPE);
    Sampled sample(stream, send_count * esize * static_cast<size_t>(comm->world_size)); // what this rank receives
    CCL_NCCL(ncclAllGather(sendbuf, recvbuf, send_count, dt, comm->comm, cudaStreamOf(stream)));
    sample.launched();
    return INFINI_STATUS_SUCCESS;
}

// One group of world_size broadcasts: root r sends its recv_counts[r] elements into everybody's slice r.
__INFINI_C infiniStatus_t infinicclAllGatherV(void *sendbuf, void *recvbuf, const size_t *recv_counts, int nranks, infiniDtype_t datatype,
                                              infinicclComm_t comm, infinirtStream_t stream) {
    CCL_REQUIRE(comm != nullptr && recv_counts != nullptr, INFINI_STATUS_NULL_POINTER);
    ncclDataType_t dt;
    size_t esize;
    CCL_REQUIRE(toNccl(datatype, &dt, &esize), INFINI_STATUS_BAD_TENSOR_DTYPE);
    CCL_REQUIRE(nranks == comm->world_size, INFINI_STATUS_BAD_PARAM);
    char *dst = static_cast<char *>(recvbuf);
    uint64_t total = 0;
    for (int r = 0; r < nranks; ++r) {
        total += recv_counts[r] * esize;
    }
    Sampled sample(stream, total);
    CCL_NCCL(ncclGroupStart());
    for (int root = 0; root < nranks; ++root) {
        const ncclResult_t r = ncclBroadcast(sendbuf, dst, recv_counts[root], dt, root, comm->comm, cudaStreamOf(stream));
        if (r != ncclSuccess) {
            (void)ncclGroupEnd();
            return fromNccl(r, "ncclBroadcast (all-gather-v)");
        }
        dst += recv_counts[root] * esize;
    }
    CCL_NCCL(ncclGroupEnd());
    sample.launched();
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infinicclReduceScatter(void *sendbuf, void *recvbuf, size_t recv_count, infiniDtype_t datatype,
                                                 infinicclReduceOp_t op, infinicclComm_t comm, infinirtStream_t stream) {
    CCL_REQUIRE(comm != nullptr, INFINI_STATUS_NULL_POINTER);
    ncclDataType_t dt;
    size_t esize;
    ncclRedOp_t rop;
    CCL_REQUIRE(toNccl(datatype, &dt, &esize), INFINI_STATUS_BAD_TENSOR_DTYPE);
    CCL_REQUIRE(toNccl(op, &rop), INFINI_STATUS_BAD_PARAM);
    Sampled sample(stream, recv_count * esize * static_cast<size_t>(comm->world_size)); // what this rank contributes
    CCL_NCCL(ncclReduceScatter(sendbuf, recvbuf, recv_count, dt, rop, comm->comm, cudaStreamOf(stream)));
    sample.launched();
    return INFINI_STATUS_SUCCESS;
}

// One group of world_size reductions: slice r of everybody's sendbuf is reduced onto rank r.
__INFINI_C infiniStatus_t infinicclReduceScatterV(void *sendbuf, void *recvbuf, const size_t *send_counts, int nranks, infiniDtype_t datatype,
                                                  infinicclReduceOp_t op, infinicclComm_t comm, infinirtStream_t stream) {
    CCL_REQUIRE(comm != nullptr && send_counts != nullptr, INFINI_STATUS_NULL_POINTER);
    ncclDataType_t dt;
    size_t esize;
    ncclRedOp_t rop;
    CCL_REQUIRE(toNccl(datatype, &dt, &esize), INFINI_STATUS_BAD_TENSOR_DTYPE);
    CCL_REQUIRE(toNccl(op, &rop), INFINI_STATUS_BAD_PARAM);
    CCL_REQUIRE(nranks == comm->world_size, INFINI_STATUS_BAD_PARAM);
    const char *src = static_cast<const char *>(sendbuf);
    uint64_t total = 0;
    for (int r = 0; r < nranks; ++r) {
        total += send_counts[r] * esize;
    }
    Sampled sample(stream, total);
    CCL_NCCL(ncclGroupStart());
    for (int root = 0; root < nranks; ++root) {
        const ncclResult_t r = ncclReduce(src, recvbuf, send_counts[root], dt, rop, root, comm->comm, cudaStreamOf(stream));
        if (r != ncclSuccess) {
            (void)ncclGroupEnd();
            return fromNccl(r, "ncclReduce (reduce-scatter-v)");
        }
        src += send_counts[root] * esize;
    }
    CCL_NCCL(ncclGroupEnd());
    sample.launched();
    return INFINI_STATUS_SUCCESS;
}
