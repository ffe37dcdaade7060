// infiniopPagedAttentionStaticWorkspace: paged-attention decode for callers that have no device
// memory of their own to offer as workspace.
//
// Who that is: a serving engine that hands every free byte of HBM to its KV block pool at start-up
// (a later cudaMalloc simply fails), a process whose device allocator is frozen once serving
// begins, or a host framework's operator callback that may only touch buffers the framework
// registered.  Such callers can still pass inputs and outputs, but cannot size and allocate the
// scratch that infiniopPagedAttention asks for through infiniopGetPagedAttentionWorkspaceSize.
//
// Here the scratch lives in this library's own image: a file-scope __device__ array of
// INFINIOP_PAGED_ATTENTION_STATIC_WORKSPACE_BYTES (32 MiB).  A GPU holds that array from the moment the
// CUDA runtime loads this file's device code on it until the process exits.  With lazy module loading
// (the runtime's default) that moment is the first call of this entry point on that device, not the
// loading of the library: the 32 MiB are taken from the device's free memory THEN.  The split-KV records, the plan
// and the combine tasks of the streaming kernels are placed in it exactly as they would be in a
// caller's buffer - the call below forwards to infiniopPagedAttention with the array's device
// address as the workspace - so results are identical to the regular entry point's.
//
// Limits and rules:
//  * a descriptor whose workspace need exceeds the array is refused with
//    INFINI_STATUS_INSUFFICIENT_WORKSPACE and a message on stderr; nothing is launched;
//  * the first call on each device looks the array's device address up (cudaGetSymbolAddress, with
//    that device current), which is also what makes the runtime place the array on that device.  Make
//    that first call at start-up - before the KV pool takes the rest of the device's memory (otherwise
//    it fails with INFINI_STATUS_INTERNAL_ERROR for want of 32 MiB) and before any stream capture
//    begins.  Later calls take no memory at all;
//  * all calls on one device share the one array.  It keeps whatever the previous call left in it;
//    that is harmless, because the kernels rewrite every field they later read (nothing in the
//    workspace has to start at zero).  Two calls that overlap on the GPU - different streams, or
//    several host threads - race on it: serialise them, or use infiniopPagedAttention with separate
//    workspaces;
//  * no cudaMalloc, cudaFree or other allocating routine is called on this path.
#include "../common.h"

#include <mutex>

namespace {

// In host code this name is only a handle for the symbol API, never a device address.
static __device__ __align__(256) unsigned char g_paged_attention_scratch[INFINIOP_PAGED_ATTENTION_STATIC_WORKSPACE_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void *g_scratch_address[kMaxDevices] = {};

// Device address of the array on the current device; looked up once per device.
infiniStatus_t scratchAddress(void **ptr) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void)cudaGetLastError();
        return INFINI_STATUS_DEVICE_NOT_FOUND;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void *address = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&address, g_paged_attention_scratch);
        if (err != cudaSuccess || address == nullptr) {
            (void)cudaGetLastError();
            std::fprintf(stderr, "[infiniop] cudaGetSymbolAddress(static paged-attention workspace) on device %d: %s\n",
                         device, cudaGetErrorString(err));
            return INFINI_STATUS_INTERNAL_ERROR;
        }
        g_scratch_address[device] = address;
    }
    *ptr = g_scratch_address[device];
    return INFINI_STATUS_SUCCESS;
}

} // namespace

__INFINI_C infiniStatus_t infiniopPagedAttentionStaticWorkspace(
    infiniopPagedAttentionDescriptor_t desc,
    void *out,
    const void *q,
    const void *k_cache,
    const void *v_cache,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    void *stream) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    size_t need = 0;
    infiniStatus_t st = infiniopGetPagedAttentionWorkspaceSize(desc, &need);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    if (need > INFINIOP_PAGED_ATTENTION_STATIC_WORKSPACE_BYTES) {
        std::fprintf(stderr,
                     "[infiniop] infiniopPagedAttentionStaticWorkspace: this problem needs %zu bytes of workspace, the built-in "
                     "array holds %u; use infiniopPagedAttention with a caller-provided workspace\n",
                     need, INFINIOP_PAGED_ATTENTION_STATIC_WORKSPACE_BYTES);
        return INFINI_STATUS_INSUFFICIENT_WORKSPACE;
    }
    void *scratch = nullptr;
    if (need > 0) {
        st = scratchAddress(&scratch);
        B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    }
    return infiniopPagedAttention(desc, scratch, need > 0 ? INFINIOP_PAGED_ATTENTION_STATIC_WORKSPACE_BYTES : 0,
                                  out, q, k_cache, v_cache, block_tables, seq_lens, alibi_slopes, stream);
}
