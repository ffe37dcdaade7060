// Internal definitions shared by the translation units of libinfiniop.
//
// The three structs that callers can see through the C ABI keep the reference's leading
// fields (reference src/infiniop/handle.h:6-9, src/infiniop/operator.h:6-9); everything
// behind them is private to this library.
#ifndef INFINIOP_B200_COMMON_H
#define INFINIOP_B200_COMMON_H

#include "infiniop.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <memory>
#include <vector>

struct InfiniopHandle {
    infiniDevice_t device;
    int device_id;
};

struct InfiniopDescriptor {
    infiniDevice_t device_type;
    int device_id;
};

struct InfiniopTensorDescriptor {
    infiniDtype_t dtype;
    std::vector<size_t> shape;
    std::vector<ptrdiff_t> strides; // in elements

    size_t ndim() const { return shape.size(); }
    size_t dim(size_t i) const { return shape[i]; }
    ptrdiff_t stride(size_t i) const { return strides[i]; }
};

namespace b200 {

// Device limits cached once per handle (the reference caches warp size / block and grid
// limits, src/infiniop/devices/nvidia/nvidia_common.cu:15-33; this path additionally needs
// the SM count and the opt-in shared memory size to size persistent grids).
struct DeviceProps {
    int device_id = 0;
    int cc_major = 0;
    int cc_minor = 0;
    int sm_count = 0;
    int max_threads_per_block = 0;
    int warp_size = 0;
    size_t smem_per_block_optin = 0;
    size_t smem_per_sm = 0;
    unsigned int *kernel_flags = nullptr; // the device's word of kernel status flags (infiniopGetKernelStatus)
};

// Device address of that word on `device_id`, which must be the current device the first time.
infiniStatus_t kernelFlagsAddress(int device_id, unsigned int **ptr);

struct Handle {
    // must stay first: callers read {device, device_id}
    InfiniopHandle base;
    std::shared_ptr<const DeviceProps> props;
};

inline size_t dtypeSize(infiniDtype_t dt) {
    switch (dt) {
    case INFINI_DTYPE_BYTE:
    case INFINI_DTYPE_BOOL:
    case INFINI_DTYPE_I8:
    case INFINI_DTYPE_U8:
    case INFINI_DTYPE_F8:
        return 1;
    case INFINI_DTYPE_I16:
    case INFINI_DTYPE_U16:
    case INFINI_DTYPE_F16:
    case INFINI_DTYPE_BF16:
        return 2;
    case INFINI_DTYPE_I32:
    case INFINI_DTYPE_U32:
    case INFINI_DTYPE_F32:
        return 4;
    case INFINI_DTYPE_I64:
    case INFINI_DTYPE_U64:
    case INFINI_DTYPE_F64:
        return 8;
    default:
        return 0;
    }
}

// Kinds of operator descriptor this library hands out; stored right after the two ABI ints
// so the generic Destroy/dispatch code can tell them apart without RTTI.
enum class OpKind : int {
    PagedAttention = 1,
    PagedCaching = 2,
    PagedAttentionPrefill = 3,
    PagedDecodeStep = 4,
    RoPE = 5,
    KVCaching = 6,
};

struct OpDescriptorBase {
    infiniDevice_t device_type;
    int device_id;
    OpKind kind;
    std::shared_ptr<const DeviceProps> props;
};

#define B200_RETURN_IF(cond, status) \
    do {                             \
        if (cond) {                  \
            return (status);         \
        }                            \
    } while (0)

inline infiniStatus_t checkLaunch(const char *what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        std::fprintf(stderr, "[infiniop] %s: %s\n", what, cudaGetErrorString(err));
        return INFINI_STATUS_INTERNAL_ERROR;
    }
    return INFINI_STATUS_SUCCESS;
}

} // namespace b200

#endif
