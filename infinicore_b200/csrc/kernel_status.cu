// The per-device word of status flags that this library's kernels raise (a wait that ran out, an index
// outside the pool in checked mode) and infiniopGetKernelStatus, which reads and clears it.
//
// The word is a file-scope __device__ variable.  In host code its name is only a handle for the symbol
// API; kernels in other translation units receive its device address (looked up here once per device,
// when the device's first handle is created) through DeviceProps::kernel_flags.
#include "common.h"

#include <mutex>

namespace {

static __device__ unsigned int g_kernel_flags = 0;

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned int *g_address[kMaxDevices] = {};

} // namespace

namespace b200 {

infiniStatus_t kernelFlagsAddress(int device_id, unsigned int **ptr) {
    B200_RETURN_IF(device_id < 0 || device_id >= kMaxDevices, INFINI_STATUS_DEVICE_NOT_FOUND);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_address[device_id] == nullptr) {
        int current = -1;
        B200_RETURN_IF(cudaGetDevice(&current) != cudaSuccess || current != device_id, INFINI_STATUS_BAD_PARAM);
        void *address = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&address, g_kernel_flags);
        if (err != cudaSuccess || address == nullptr) {
            (void)cudaGetLastError();
            std::fprintf(stderr, "[infiniop] cudaGetSymbolAddress(kernel status word) on device %d: %s\n", device_id,
                         cudaGetErrorString(err));
            return INFINI_STATUS_INTERNAL_ERROR;
        }
        g_address[device_id] = static_cast<unsigned int *>(address);
    }
    *ptr = g_address[device_id];
    return INFINI_STATUS_SUCCESS;
}

} // namespace b200

__INFINI_C infiniStatus_t infiniopGetKernelStatus(infiniopHandle_t handle, void *stream, unsigned int *flags) {
    B200_RETURN_IF(handle == nullptr || flags == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(handle->device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);
    const auto *h = reinterpret_cast<const b200::Handle *>(handle);
    unsigned int *word = h->props->kernel_flags;
    B200_RETURN_IF(word == nullptr, INFINI_STATUS_INTERNAL_ERROR);
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        return b200::checkLaunch("infiniopGetKernelStatus: stream");
    }
    unsigned int value = 0;
    if (cudaMemcpy(&value, word, sizeof(value), cudaMemcpyDeviceToHost) != cudaSuccess) {
        return b200::checkLaunch("infiniopGetKernelStatus: read");
    }
    if (value != 0 && cudaMemset(word, 0, sizeof(value)) != cudaSuccess) {
        return b200::checkLaunch("infiniopGetKernelStatus: clear");
    }
    *flags = value;
    return INFINI_STATUS_SUCCESS;
}
