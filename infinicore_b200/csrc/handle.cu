// Handle, tensor-descriptor and operator-descriptor entry points of libinfiniop.
//
// Behaviour follows reference src/infiniop/devices/handle.cc:26-128 (handle bound to the
// calling thread's current infinirt device), src/infiniop/tensor_descriptor.cc:8-29
// (NULL strides => row-major contiguous) and src/infiniop/operator_descriptor.cc:3-15.
// There is exactly one backend: an NVIDIA device of compute capability 10.x.
#include "common.h"
#include "infinirt.h"

using b200::DeviceProps;
using b200::Handle;

__INFINI_C infiniStatus_t infiniopCreateHandle(infiniopHandle_t *handle_ptr) {
    B200_RETURN_IF(handle_ptr == nullptr, INFINI_STATUS_NULL_POINTER);

    infiniDevice_t device = INFINI_DEVICE_CPU;
    int device_id = 0;
    infiniStatus_t st = infinirtGetDevice(&device, &device_id);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    B200_RETURN_IF(device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);

    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_id) != cudaSuccess) {
        (void)cudaGetLastError();
        return INFINI_STATUS_DEVICE_NOT_FOUND;
    }
    if (prop.major != 10) {
        std::fprintf(stderr,
                     "[infiniop] device %d is sm_%d%d; this library carries sm_100a code only\n",
                     device_id, prop.major, prop.minor);
        return INFINI_STATUS_DEVICE_ARCHITECTURE_NOT_SUPPORTED;
    }

    auto props = std::make_shared<DeviceProps>();
    props->device_id = device_id;
    props->cc_major = prop.major;
    props->cc_minor = prop.minor;
    props->sm_count = prop.multiProcessorCount;
    props->max_threads_per_block = prop.maxThreadsPerBlock;
    props->warp_size = prop.warpSize;
    props->smem_per_block_optin = prop.sharedMemPerBlockOptin;
    props->smem_per_sm = prop.sharedMemPerMultiprocessor;
    st = b200::kernelFlagsAddress(device_id, &props->kernel_flags);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);

    auto *h = new Handle{{device, device_id}, std::move(props)};
    *handle_ptr = reinterpret_cast<infiniopHandle_t>(h);
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopDestroyHandle(infiniopHandle_t handle) {
    B200_RETURN_IF(handle == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(handle->device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);
    delete reinterpret_cast<Handle *>(handle);
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopCreateTensorDescriptor(
    infiniopTensorDescriptor_t *desc_ptr,
    size_t ndim,
    const size_t *shape,
    const ptrdiff_t *strides,
    infiniDtype_t dtype) {
    B200_RETURN_IF(desc_ptr == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(ndim > 0 && shape == nullptr, INFINI_STATUS_NULL_POINTER);

    auto *d = new InfiniopTensorDescriptor();
    d->dtype = dtype;
    d->shape.assign(shape, shape + ndim);
    if (strides != nullptr) {
        d->strides.assign(strides, strides + ndim);
    } else {
        d->strides.resize(ndim);
        ptrdiff_t running = 1;
        for (size_t i = ndim; i-- > 0;) {
            d->strides[i] = running;
            running *= static_cast<ptrdiff_t>(shape[i]);
        }
    }
    *desc_ptr = d;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopDestroyTensorDescriptor(infiniopTensorDescriptor_t desc) {
    delete desc;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopGetDescriptorDeviceType(
    const struct InfiniopDescriptor *desc_ptr, infiniDevice_t *device_type) {
    B200_RETURN_IF(desc_ptr == nullptr || device_type == nullptr, INFINI_STATUS_NULL_POINTER);
    *device_type = desc_ptr->device_type;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopGetDescriptorDeviceId(
    const struct InfiniopDescriptor *desc_ptr, int *device_id) {
    B200_RETURN_IF(desc_ptr == nullptr || device_id == nullptr, INFINI_STATUS_NULL_POINTER);
    *device_id = desc_ptr->device_id;
    return INFINI_STATUS_SUCCESS;
}
