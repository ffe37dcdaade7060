// infiniopPagedCaching: scatter of new K/V rows into the paged cache pools.
//
// Semantics follow reference src/infiniop/ops/paged_caching/info.h:35-107 (accepted
// dtypes/shapes, which strides are captured) and
// src/infiniop/ops/paged_caching/cuda/kernel.cuh:55-88 (slot -> (block, offset), negative
// slot skipped, K and V copied element for element).  The copy is a pure byte move, so the
// result is bit-exact for every dtype.
//
// Kernel shape: a row is head_size * sizeof(T) contiguous bytes on both sides (last-dim stride
// is 1).  When the row lengths, the base pointers and all strides are 16-byte multiples it is
// cut into 128-bit words, otherwise into elements; one thread moves word i of the K row and of
// the V row of one (token, kv-head), consecutive threads consecutive words.  In a decode step the
// workload is tiny (config "Llama-3-8B decode": 64 tokens x 8 heads x 256 B x {K,V} = 256 KiB in,
// 256 KiB out) and launch-latency bound; after a prefill it is tens of thousands of tokens and
// HBM-bound.  The grid is sized to the word count.
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
    bool check_indices; // INFINIOP_PAGED_CHECK_INDICES (default 0), likewise
    size_t num_blocks;
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
    long long num_pairs; // num_tokens * num_kv_heads: a K row and a V row each
    int items_per_pair;  // words of the longer of the two rows
    int small;           // num_pairs * items_per_pair (rounded up to whole blocks) fits 32 bits
    int num_kv_heads;
    int block_size;
    int k_row_bytes;
    int v_row_bytes;
    long long k_src_token, k_src_head, v_src_token, v_src_head;
    long long k_blk, k_head, k_slot, v_blk, v_head, v_slot;
    // index checking (INFINIOP_PAGED_CHECK_INDICES=1 when the descriptor was created): a slot at or beyond
    // num_slots raises INFINIOP_KERNEL_FLAG_SLOT_OUT_OF_RANGE in the device's status word and its row is
    // skipped; unchecked, the row goes wherever the slot says, as in the reference's kernel
    // (src/infiniop/ops/paged_caching/cuda/kernel.cuh:60-78)
    unsigned int *kernel_flags;
    long long num_slots;
    int check_indices;
};

constexpr int kThreads = 128;

// One thread per item of a (token, kv-head) pair: item i is the i-th Vec-sized word of the K row and of the
// V row (a thread skips the side whose row is shorter than i words).  Consecutive threads take consecutive
// words, so a warp covers whole rows with 128-bit accesses and both loads are in flight before the first
// store.  The same kernel serves a decode step (64 tokens, launch-latency bound) and a prefill-sized scatter
// (tens of thousands of tokens, HBM-bound).
template <typename Vec>
__global__ void __launch_bounds__(kThreads) pagedCachingScatterKernel(const KernelArgs a) {
    // Launched with the programmatic-serialization attribute: wait for the preceding kernel in the
    // stream (which may still be reading the pools or producing k/v), then let the next one start
    // its prologue.  Both are no-ops for a normal launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    long long pair, token;
    int item, head;
    if (a.small) {
        // fewer than 2^32 items: 32-bit divisions (a 64-bit one costs several times as much)
        const unsigned idx = blockIdx.x * static_cast<unsigned>(kThreads) + threadIdx.x;
        const unsigned pr = idx / static_cast<unsigned>(a.items_per_pair);
        const unsigned tk = pr / static_cast<unsigned>(a.num_kv_heads);
        item = static_cast<int>(idx - pr * a.items_per_pair);
        head = static_cast<int>(pr - tk * a.num_kv_heads);
        pair = pr;
        token = tk;
    } else {
        const long long idx = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
        pair = idx / a.items_per_pair;
        item = static_cast<int>(idx - pair * a.items_per_pair);
        head = static_cast<int>(pair % a.num_kv_heads);
        token = pair / a.num_kv_heads;
    }
    if (pair >= a.num_pairs) {
        return;
    }
    const int64_t slot = a.slot_mapping[token];
    if (slot < 0) {
        return; // padding token
    }
    if (a.check_indices && slot >= a.num_slots) {
        if (item == 0 && head == 0) {
            atomicOr(a.kernel_flags, 4u);
        }
        return;
    }
    long long block, off;
    if (slot <= 0x7fffffffLL) {
        const unsigned s32 = static_cast<unsigned>(slot);
        const unsigned blk = s32 / static_cast<unsigned>(a.block_size);
        block = blk;
        off = s32 - blk * static_cast<unsigned>(a.block_size);
    } else {
        block = slot / a.block_size;
        off = slot % a.block_size;
    }
    const long long byte = static_cast<long long>(item) * static_cast<long long>(sizeof(Vec));
    const bool has_k = byte < a.k_row_bytes;
    const bool has_v = byte < a.v_row_bytes;
    Vec k_item{}, v_item{};
    if (has_k) {
        k_item = *reinterpret_cast<const Vec *>(a.k + token * a.k_src_token + head * a.k_src_head + byte);
    }
    if (has_v) {
        v_item = *reinterpret_cast<const Vec *>(a.v + token * a.v_src_token + head * a.v_src_head + byte);
    }
    if (has_k) {
        *reinterpret_cast<Vec *>(a.k_cache + block * a.k_blk + head * a.k_head + off * a.k_slot + byte) = k_item;
    }
    if (has_v) {
        *reinterpret_cast<Vec *>(a.v_cache + block * a.v_blk + head * a.v_head + off * a.v_slot + byte) = v_item;
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
    a.num_pairs = static_cast<long long>(I.num_tokens) * static_cast<long long>(I.num_kv_heads);
    a.num_kv_heads = static_cast<int>(I.num_kv_heads);
    a.block_size = static_cast<int>(I.block_size);
    a.kernel_flags = desc.base.props->kernel_flags;
    a.num_slots = static_cast<long long>(desc.num_blocks) * static_cast<long long>(I.block_size);
    a.check_indices = (desc.check_indices && a.kernel_flags != nullptr) ? 1 : 0;
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

    auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec16 = I.strides_vec16 && aligned16(k_cache) && aligned16(v_cache) && aligned16(k) && aligned16(v);
    const int word = vec16 ? 16 : static_cast<int>(I.elem_size);
    const int longer = a.k_row_bytes > a.v_row_bytes ? a.k_row_bytes : a.v_row_bytes;
    a.items_per_pair = longer / word;
    if (a.items_per_pair == 0) {
        return INFINI_STATUS_SUCCESS; // rows of zero width
    }
    const long long blocks = (a.num_pairs * a.items_per_pair + kThreads - 1) / kThreads;
    B200_RETURN_IF(blocks > 0x7fffffffLL, INFINI_STATUS_BAD_TENSOR_SHAPE);
    a.small = blocks * kThreads <= 0xffffffffLL ? 1 : 0;
    const dim3 grid(static_cast<unsigned>(blocks));
    const dim3 block(kThreads);

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
    const char *check_env = std::getenv("INFINIOP_PAGED_CHECK_INDICES");
    const bool check = check_env != nullptr && check_env[0] == '1';
    auto *d = new Descriptor{{handle->device, handle->device_id, b200::OpKind::PagedCaching, h->props}, info, use_pdl, check,
                             k_cache_desc->dim(0)};
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
