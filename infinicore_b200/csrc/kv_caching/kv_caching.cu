// infiniopKVCaching: append new K/V rows to a contiguous [batch, kv_heads, max_seq_len, hidden] cache.
//
// Semantics follow reference src/infiniop/ops/kv_caching/info.h:22-112 (accepted dtypes and ranks, every
// stride of the four tensors captured) and src/infiniop/ops/kv_caching/cuda/kernel.cuh:32-60 (row s of
// sequence b goes to cache position past_kv_lengths[b] + s; K and V copied element for element).  A pure
// byte move, so bit-exact for every dtype.
//
// Kernel shape: HBM-bound copy.  When every last stride is 1 and all row starts are 16-byte aligned a row
// is cut into 128-bit words, consecutive threads on consecutive words, each thread moving its word of the
// K row and of the V row; otherwise a thread moves one K and one V element through the full stride set.
// Offsets are 64-bit (the reference's are int, kernel.cuh:52-57); the row decomposition uses 32-bit
// divisions when the item count allows.
#include "../common.h"

namespace b200::kv_caching {

struct Info {
    infiniDtype_t dtype, len_dtype;
    size_t elem_size;
    size_t batch, num_kv_heads, max_seq_len, seq_len, hidden;
    ptrdiff_t kc[4], vc[4], k[4], v[4]; // element strides
    bool strides_vec16;                 // last strides 1, row bytes and every other stride multiples of 16 bytes
};

struct Descriptor {
    OpDescriptorBase base;
    Info info;
};

// Strides in BYTES.
struct KernelArgs {
    unsigned char *k_cache;
    unsigned char *v_cache;
    const unsigned char *k;
    const unsigned char *v;
    const void *past_kv_lengths;
    long long rows; // batch * kv_heads * seq_len (a thread moves its item of the K row and of the V row)
    int num_kv_heads, seq_len, items_per_row;
    long long max_seq_len;
    long long kc[4], vc[4], ks[4], vs[4];
    int len_is_64;
    int small; // rows * items_per_row (rounded up to whole blocks) fits 32 bits
};

constexpr int kThreads = 256;

// Item = one 128-bit word (Vec = uint4) or one element (Vec = the element's unsigned type) of a row.  A thread
// moves the item of the K row and of the V row of one (batch, head, token): two independent loads in flight
// before the first store.
template <typename Vec, bool kDenseRows>
__global__ void __launch_bounds__(kThreads) kvCachingRowsKernel(const KernelArgs a) {
    long long row, s, h, b;
    int item;
    if (a.small) {
        // fewer than 2^32 items: 32-bit divisions (a 64-bit one costs several times as much)
        const unsigned idx = blockIdx.x * static_cast<unsigned>(kThreads) + threadIdx.x;
        const unsigned r = idx / static_cast<unsigned>(a.items_per_row);
        const unsigned bh = r / static_cast<unsigned>(a.seq_len);
        const unsigned bb = bh / static_cast<unsigned>(a.num_kv_heads);
        item = static_cast<int>(idx - r * a.items_per_row);
        row = r;
        s = r - bh * a.seq_len;
        h = bh - bb * a.num_kv_heads;
        b = bb;
    } else {
        const long long idx = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
        row = idx / a.items_per_row;
        item = static_cast<int>(idx - row * a.items_per_row);
        s = row % a.seq_len;
        h = (row / a.seq_len) % a.num_kv_heads;
        b = row / (static_cast<long long>(a.seq_len) * a.num_kv_heads);
    }
    if (row >= a.rows) {
        return;
    }
    const long long past = a.len_is_64 ? static_cast<const long long *>(a.past_kv_lengths)[b]
                                       : static_cast<long long>(static_cast<const int *>(a.past_kv_lengths)[b]);
    const long long dst_s = past + s;
    if (dst_s < 0 || dst_s >= a.max_seq_len) {
        return; // outside the cache
    }
    const long long step = static_cast<long long>(sizeof(Vec));
    const unsigned char *k_src = a.k + b * a.ks[0] + h * a.ks[1] + s * a.ks[2] + item * (kDenseRows ? step : a.ks[3]);
    const unsigned char *v_src = a.v + b * a.vs[0] + h * a.vs[1] + s * a.vs[2] + item * (kDenseRows ? step : a.vs[3]);
    unsigned char *k_dst = a.k_cache + b * a.kc[0] + h * a.kc[1] + dst_s * a.kc[2] + item * (kDenseRows ? step : a.kc[3]);
    unsigned char *v_dst = a.v_cache + b * a.vc[0] + h * a.vc[1] + dst_s * a.vc[2] + item * (kDenseRows ? step : a.vc[3]);
    const Vec k_item = *reinterpret_cast<const Vec *>(k_src);
    const Vec v_item = *reinterpret_cast<const Vec *>(v_src);
    *reinterpret_cast<Vec *>(k_dst) = k_item;
    *reinterpret_cast<Vec *>(v_dst) = v_item;
}

static infiniStatus_t makeInfo(Info &out, infiniopTensorDescriptor_t k_cache, infiniopTensorDescriptor_t v_cache,
                               infiniopTensorDescriptor_t k, infiniopTensorDescriptor_t v, infiniopTensorDescriptor_t past) {
    const infiniDtype_t dtype = k_cache->dtype;
    B200_RETURN_IF(dtype != INFINI_DTYPE_F16 && dtype != INFINI_DTYPE_BF16 && dtype != INFINI_DTYPE_F32, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(v_cache->dtype != dtype || k->dtype != dtype || v->dtype != dtype, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(past->dtype != INFINI_DTYPE_I32 && past->dtype != INFINI_DTYPE_I64, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(k_cache->ndim() != 4 || v_cache->ndim() != 4 || k->ndim() != 4 || v->ndim() != 4, INFINI_STATUS_BAD_TENSOR_SHAPE);
    for (size_t i = 0; i < 4; ++i) {
        B200_RETURN_IF(k_cache->dim(i) != v_cache->dim(i) || k->dim(i) != v->dim(i), INFINI_STATUS_BAD_TENSOR_SHAPE);
    }
    B200_RETURN_IF(k->dim(0) != k_cache->dim(0) || k->dim(1) != k_cache->dim(1) || k->dim(3) != k_cache->dim(3),
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(past->ndim() != 1 || past->dim(0) != k_cache->dim(0), INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(past->dim(0) > 1 && past->stride(0) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);

    out.dtype = dtype;
    out.len_dtype = past->dtype;
    out.elem_size = dtypeSize(dtype);
    out.batch = k_cache->dim(0);
    out.num_kv_heads = k_cache->dim(1);
    out.max_seq_len = k_cache->dim(2);
    out.hidden = k_cache->dim(3);
    out.seq_len = k->dim(2);
    B200_RETURN_IF(out.num_kv_heads > 0x7fffffffu || out.seq_len > 0x7fffffffu || out.hidden > 0x7fffffffu, INFINI_STATUS_BAD_TENSOR_SHAPE);
    for (size_t i = 0; i < 4; ++i) {
        out.kc[i] = k_cache->stride(i);
        out.vc[i] = v_cache->stride(i);
        out.k[i] = k->stride(i);
        out.v[i] = v->stride(i);
    }
    const auto mult16 = [&](ptrdiff_t elems) { return (static_cast<long long>(elems) * static_cast<long long>(out.elem_size)) % 16 == 0; };
    bool vec = mult16(static_cast<ptrdiff_t>(out.hidden));
    for (const ptrdiff_t *st : {out.kc, out.vc, out.k, out.v}) {
        vec = vec && (out.hidden == 1 || st[3] == 1) && mult16(st[0]) && mult16(st[1]) && mult16(st[2]);
    }
    out.strides_vec16 = vec;
    return INFINI_STATUS_SUCCESS;
}

} // namespace b200::kv_caching

using b200::kv_caching::Descriptor;

__INFINI_C infiniStatus_t infiniopCreateKVCachingDescriptor(
    infiniopHandle_t handle,
    infiniopKVCachingDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t k_cache,
    infiniopTensorDescriptor_t v_cache,
    infiniopTensorDescriptor_t k,
    infiniopTensorDescriptor_t v,
    infiniopTensorDescriptor_t past_kv_lengths) {
    B200_RETURN_IF(handle == nullptr || desc_ptr == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(k_cache == nullptr || v_cache == nullptr || k == nullptr || v == nullptr || past_kv_lengths == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(handle->device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);
    b200::kv_caching::Info info;
    const infiniStatus_t st = b200::kv_caching::makeInfo(info, k_cache, v_cache, k, v, past_kv_lengths);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    auto *h = reinterpret_cast<b200::Handle *>(handle);
    auto *d = new Descriptor{{handle->device, handle->device_id, b200::OpKind::KVCaching, h->props}, info};
    *desc_ptr = reinterpret_cast<infiniopKVCachingDescriptor_t>(d);
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopGetKVCachingWorkspaceSize(infiniopKVCachingDescriptor_t desc, size_t *size) {
    B200_RETURN_IF(desc == nullptr || size == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(reinterpret_cast<Descriptor *>(desc)->base.kind != b200::OpKind::KVCaching, INFINI_STATUS_BAD_PARAM);
    *size = 0;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopKVCaching(
    infiniopKVCachingDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *k_cache,
    void *v_cache,
    const void *k,
    const void *v,
    const void *past_kv_lengths,
    void *stream) {
    (void)workspace;
    (void)workspace_size;
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<Descriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::KVCaching, INFINI_STATUS_BAD_PARAM);
    const auto &I = d->info;
    const long long rows = static_cast<long long>(I.batch) * static_cast<long long>(I.num_kv_heads) * static_cast<long long>(I.seq_len);
    if (rows == 0 || I.hidden == 0 || I.max_seq_len == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    B200_RETURN_IF(k_cache == nullptr || v_cache == nullptr || k == nullptr || v == nullptr || past_kv_lengths == nullptr,
                   INFINI_STATUS_NULL_POINTER);

    const auto addr = [](const void *p) { return reinterpret_cast<uintptr_t>(p); };
    const bool vec = I.strides_vec16 && ((addr(k_cache) | addr(v_cache) | addr(k) | addr(v)) & 15u) == 0;
    b200::kv_caching::KernelArgs a{};
    a.k_cache = static_cast<unsigned char *>(k_cache);
    a.v_cache = static_cast<unsigned char *>(v_cache);
    a.k = static_cast<const unsigned char *>(k);
    a.v = static_cast<const unsigned char *>(v);
    a.past_kv_lengths = past_kv_lengths;
    a.rows = rows;
    a.num_kv_heads = static_cast<int>(I.num_kv_heads);
    a.seq_len = static_cast<int>(I.seq_len);
    a.max_seq_len = static_cast<long long>(I.max_seq_len);
    a.items_per_row = vec ? static_cast<int>(I.hidden * I.elem_size / 16) : static_cast<int>(I.hidden);
    const long long es = static_cast<long long>(I.elem_size);
    for (int i = 0; i < 4; ++i) {
        a.kc[i] = I.kc[i] * es;
        a.vc[i] = I.vc[i] * es;
        a.ks[i] = I.k[i] * es;
        a.vs[i] = I.v[i] * es;
    }
    a.len_is_64 = I.len_dtype == INFINI_DTYPE_I64 ? 1 : 0;
    const long long blocks = (rows * a.items_per_row + b200::kv_caching::kThreads - 1) / b200::kv_caching::kThreads;
    B200_RETURN_IF(blocks > 0x7fffffffLL, INFINI_STATUS_BAD_TENSOR_SHAPE);
    a.small = blocks * b200::kv_caching::kThreads <= 0xffffffffLL ? 1 : 0;

    auto cuda_stream = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>(blocks);
    using namespace b200::kv_caching;
    if (vec) {
        kvCachingRowsKernel<uint4, true><<<grid, kThreads, 0, cuda_stream>>>(a);
    } else if (I.elem_size == 2) {
        kvCachingRowsKernel<unsigned short, false><<<grid, kThreads, 0, cuda_stream>>>(a);
    } else {
        kvCachingRowsKernel<unsigned int, false><<<grid, kThreads, 0, cuda_stream>>>(a);
    }
    return b200::checkLaunch("kvCachingRowsKernel");
}

__INFINI_C infiniStatus_t infiniopDestroyKVCachingDescriptor(infiniopKVCachingDescriptor_t desc) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<Descriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::KVCaching, INFINI_STATUS_BAD_PARAM);
    delete d;
    return INFINI_STATUS_SUCCESS;
}
