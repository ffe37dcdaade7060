// infiniopPagedCaching: scatter of new K/V rows into the paged cache pools.
//
// Semantics follow reference src/infiniop/ops/paged_caching/info.h:35-107 (accepted
// dtypes/shapes, which strides are captured) and
// src/infiniop/ops/paged_caching/cuda/kernel.cuh:55-88 (slot -> (block, offset), negative
// slot skipped, K and V copied element for element).  The copy is a pure byte move, so the
// result is bit-exact for every dtype.
//
// Kernel shape: one warp moves one (token, kv-head) row of K or of V.  A row is
// head_size * sizeof(T) contiguous bytes on both sides (last-dim stride is 1), so when the
// row length, both base pointers and all strides are 16-byte multiples the warp moves it
// with 128-bit loads/stores; otherwise it falls back to element-sized accesses.  The
// workload is tiny (config "Llama-3-8B decode": 64 tokens x 8 heads x 256 B x {K,V} =
// 256 KiB in, 256 KiB out) and launch-latency bound; the grid is sized to the row count.
#include "../common.h"

#include <cstdlib>
#include <cstring>

namespace b200::paged_caching {

struct Info {
    infiniDtype_t dtype;
    size_t elem_size;
    size_t num_tokens;
    size_t num_kv_heads;
    size_t head_size;
    size_t v_head_size;
    size_t block_size;
    // element strides
    ptrdiff_t k_src_token_stride, k_src_head_stride;
    ptrdiff_t v_src_token_stride, v_src_head_stride;
    ptrdiff_t k_cache_block_stride, k_cache_head_stride, k_cache_slot_stride;
    ptrdiff_t v_cache_block_stride, v_cache_head_stride, v_cache_slot_stride;
    bool strides_vec16; // every stride and both row lengths are multiples of 16 bytes
};

struct Descriptor {
    OpDescriptorBase base;
    Info info;
    bool use_pdl; // INFINIOP_PAGED_DECODE_PDL (default 1), read when the descriptor is created
};

static infiniStatus_t makeInfo(Info &out,
                               infiniopTensorDescriptor_t k_cache_desc,
                               infiniopTensorDescriptor_t v_cache_desc,
                               infiniopTensorDescriptor_t k_desc,
                               infiniopTensorDescriptor_t v_desc,
                               infiniopTensorDescriptor_t slot_mapping_desc) {
    const infiniDtype_t dtype = k_desc->dtype;
    B200_RETURN_IF(dtype != INFINI_DTYPE_F16 && dtype != INFINI_DTYPE_BF16 && dtype != INFINI_DTYPE_F32,
                   INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(v_desc->dtype != dtype || k_cache_desc->dtype != dtype || v_cache_desc->dtype != dtype,
                   INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(slot_mapping_desc->dtype != INFINI_DTYPE_I64, INFINI_STATUS_BAD_TENSOR_DTYPE);

    B200_RETURN_IF(k_desc->ndim() != 3 || v_desc->ndim() != 3, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(k_cache_desc->ndim() < 4 || v_cache_desc->ndim() < 4, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(slot_mapping_desc->ndim() != 1, INFINI_STATUS_BAD_TENSOR_SHAPE);

    out.dtype = dtype;
    out.elem_size = dtypeSize(dtype);
    out.num_tokens = slot_mapping_desc->dim(0);
    out.num_kv_heads = k_desc->dim(1);
    out.head_size = k_desc->dim(2);
    out.v_head_size = v_desc->dim(2);
    out.block_size = k_cache_desc->dim(2);

    B200_RETURN_IF(k_desc->dim(0) != out.num_tokens || v_desc->dim(0) != out.num_tokens || v_desc->dim(1) != out.num_kv_heads,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(v_cache_desc->dim(0) != k_cache_desc->dim(0) || v_cache_desc->dim(1) != out.num_kv_heads || v_cache_desc->dim(2) != out.block_size,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(k_cache_desc->dim(1) != out.num_kv_heads || k_cache_desc->dim(3) != out.head_size || v_cache_desc->dim(3) != out.v_head_size,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(out.block_size == 0, INFINI_STATUS_BAD_TENSOR_SHAPE);

    // Rows are moved as contiguous byte runs.
    B200_RETURN_IF(out.head_size > 1 && (k_desc->stride(2) != 1 || k_cache_desc->stride(3) != 1), INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF(out.v_head_size > 1 && (v_desc->stride(2) != 1 || v_cache_desc->stride(3) != 1), INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF(out.num_tokens > 1 && slot_mapping_desc->stride(0) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);

    out.k_src_token_stride = k_desc->stride(0);
    out.k_src_head_stride = k_desc->stride(1);
    out.v_src_token_stride = v_desc->stride(0);
    out.v_src_head_stride = v_desc->stride(1);
    out.k_cache_block_stride = k_cache_desc->stride(0);
    out.k_cache_head_stride = k_cache_desc->stride(1);
    out.k_cache_slot_stride = k_cache_desc->stride(2);
    out.v_cache_block_stride = v_cache_desc->stride(0);
    out.v_cache_head_stride = v_cache_desc->stride(1);
    out.v_cache_slot_stride = v_cache_desc->stride(2);

    auto mult16 = [&](ptrdiff_t elems) { return (static_cast<long long>(elems) * static_cast<long long>(out.elem_size)) % 16 == 0; };
    out.strides_vec16 = mult16(static_cast<ptrdiff_t>(out.head_size)) && mult16(static_cast<ptrdiff_t>(out.v_head_size))
                     && mult16(out.k_src_token_stride) && mult16(out.k_src_head_stride)
                     && mult16(out.v_src_token_stride) && mult16(out.v_src_head_stride)
                     && mult16(out.k_cache_block_stride) && mult16(out.k_cache_head_stride) && mult16(out.k_cache_slot_stride)
                     && mult16(out.v_cache_block_stride) && mult16(out.v_cache_head_stride) && mult16(out.v_cache_slot_stride);
    return INFINI_STATUS_SUCCESS;
}

// Strides below are in BYTES.
struct KernelArgs {
    unsigned char *k_cache;
    unsigned char *v_cache;
    const unsigned char *k;
    const unsigned char *v;
    const int64_t *slot_mapping;
    long long num_rows; // num_tokens * num_kv_heads * 2 (K rows then V rows interleaved per (token, head))
    int num_kv_heads;
    int block_size;
    int k_row_bytes;
    int v_row_bytes;
    long long k_src_token, k_src_head, v_src_token, v_src_head;
    long long k_blk, k_head, k_slot, v_blk, v_head, v_slot;
};

constexpr int kWarpsPerBlock = 8;

template <typename Vec>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    pagedCachingScatterKernel(const KernelArgs a) {
    // Launched with the programmatic-serialization attribute: wait for the preceding kernel in the
    // stream (which may still be reading the pools or producing k/v), then let the next one start
    // its prologue.  Both are no-ops for a normal launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= a.num_rows) {
        return;
    }
    const int lane = threadIdx.x & 31;
    const int is_v = static_cast<int>(row & 1);
    const long long th = row >> 1;
    const int head = static_cast<int>(th % a.num_kv_heads);
    const long long token = th / a.num_kv_heads;

    const int64_t slot = a.slot_mapping[token];
    if (slot < 0) {
        return; // padding token
    }
    const int64_t block = slot / a.block_size;
    const int64_t off = slot % a.block_size;

    const unsigned char *src;
    unsigned char *dst;
    int bytes;
    if (is_v) {
        src = a.v + token * a.v_src_token + head * a.v_src_head;
        dst = a.v_cache + block * a.v_blk + head * a.v_head + off * a.v_slot;
        bytes = a.v_row_bytes;
    } else {
        src = a.k + token * a.k_src_token + head * a.k_src_head;
        dst = a.k_cache + block * a.k_blk + head * a.k_head + off * a.k_slot;
        bytes = a.k_row_bytes;
    }
    const int n = bytes / static_cast<int>(sizeof(Vec));
    const Vec *s = reinterpret_cast<const Vec *>(src);
    Vec *d = reinterpret_cast<Vec *>(dst);
    for (int i = lane; i < n; i += 32) {
        d[i] = s[i];
    }
}

static infiniStatus_t launch(const Descriptor &desc,
                             void *k_cache, void *v_cache, const void *k, const void *v,
                             const void *slot_mapping, cudaStream_t stream) {
    const Info &I = desc.info;
    if (I.num_tokens == 0 || I.num_kv_heads == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    const long long es = static_cast<long long>(I.elem_size);
    KernelArgs a;
    a.k_cache = static_cast<unsigned char *>(k_cache);
    a.v_cache = static_cast<unsigned char *>(v_cache);
    a.k = static_cast<const unsigned char *>(k);
    a.v = static_cast<const unsigned char *>(v);
    a.slot_mapping = static_cast<const int64_t *>(slot_mapping);
    a.num_rows = static_cast<long long>(I.num_tokens) * static_cast<long long>(I.num_kv_heads) * 2;
    a.num_kv_heads = static_cast<int>(I.num_kv_heads);
    a.block_size = static_cast<int>(I.block_size);
    a.k_row_bytes = static_cast<int>(I.head_size * I.elem_size);
    a.v_row_bytes = static_cast<int>(I.v_head_size * I.elem_size);
    a.k_src_token = I.k_src_token_stride * es;
    a.k_src_head = I.k_src_head_stride * es;
    a.v_src_token = I.v_src_token_stride * es;
    a.v_src_head = I.v_src_head_stride * es;
    a.k_blk = I.k_cache_block_stride * es;
    a.k_head = I.k_cache_head_stride * es;
    a.k_slot = I.k_cache_slot_stride * es;
    a.v_blk = I.v_cache_block_stride * es;
    a.v_head = I.v_cache_head_stride * es;
    a.v_slot = I.v_cache_slot_stride * es;

    const long long blocks = (a.num_rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    B200_RETURN_IF(blocks > 0x7fffffffLL, INFINI_STATUS_BAD_TENSOR_SHAPE);
    const dim3 grid(static_cast<unsigned>(blocks));
    const dim3 block(kWarpsPerBlock * 32);

    auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec16 = I.strides_vec16 && aligned16(k_cache) && aligned16(v_cache) && aligned16(k) && aligned16(v);
    cudaLaunchAttribute pdl;
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl.val.programmaticStreamSerializationAllowed = desc.use_pdl ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cfg.attrs = &pdl;
    cfg.numAttrs = 1;
    cudaError_t err;
    if (vec16) {
        err = cudaLaunchKernelEx(&cfg, pagedCachingScatterKernel<uint4>, a);
    } else if (I.elem_size == 4) {
        err = cudaLaunchKernelEx(&cfg, pagedCachingScatterKernel<uint32_t>, a);
    } else {
        err = cudaLaunchKernelEx(&cfg, pagedCachingScatterKernel<uint16_t>, a);
    }
    (void)err;
    return checkLaunch("pagedCachingScatterKernel");
}

} // namespace b200::paged_caching

using b200::paged_caching::Descriptor;

__INFINI_C infiniStatus_t infiniopCreatePagedCachingDescriptor(
    infiniopHandle_t handle,
    infiniopPagedCachingDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t k_desc,
    infiniopTensorDescriptor_t v_desc,
    infiniopTensorDescriptor_t slot_mapping_desc) {
    B200_RETURN_IF(handle == nullptr || desc_ptr == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(k_cache_desc == nullptr || v_cache_desc == nullptr || k_desc == nullptr || v_desc == nullptr || slot_mapping_desc == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(handle->device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);

    b200::paged_caching::Info info;
    infiniStatus_t st = b200::paged_caching::makeInfo(info, k_cache_desc, v_cache_desc, k_desc, v_desc, slot_mapping_desc);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);

    auto *h = reinterpret_cast<b200::Handle *>(handle);
    const char *pdl_env = std::getenv("INFINIOP_PAGED_DECODE_PDL");
    const bool use_pdl = !(pdl_env != nullptr && pdl_env[0] == '0');
    auto *d = new Descriptor{{handle->device, handle->device_id, b200::OpKind::PagedCaching, h->props}, info, use_pdl};
    *desc_ptr = reinterpret_cast<infiniopPagedCachingDescriptor_t>(d);
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopGetPagedCachingWorkspaceSize(
    infiniopPagedCachingDescriptor_t desc, size_t *size) {
    B200_RETURN_IF(desc == nullptr || size == nullptr, INFINI_STATUS_NULL_POINTER);
    *size = 0;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopPagedCaching(
    infiniopPagedCachingDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *k_cache,
    void *v_cache,
    const void *k,
    const void *v,
    const void *slot_mapping,
    void *stream) {
    (void)workspace;
    (void)workspace_size;
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<Descriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::PagedCaching, INFINI_STATUS_BAD_PARAM);
    if (d->info.num_tokens == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    B200_RETURN_IF(k_cache == nullptr || v_cache == nullptr || k == nullptr || v == nullptr || slot_mapping == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    return b200::paged_caching::launch(*d, k_cache, v_cache, k, v, slot_mapping, static_cast<cudaStream_t>(stream));
}

__INFINI_C infiniStatus_t infiniopDestroyPagedCachingDescriptor(
    infiniopPagedCachingDescriptor_t desc) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    delete reinterpret_cast<Descriptor *>(desc);
    return INFINI_STATUS_SUCCESS;
}
