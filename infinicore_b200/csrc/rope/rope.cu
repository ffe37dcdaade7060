// infiniopRoPE: rotary position embedding over [seqlen, nhead, dhead] or [batch, seqlen, nhead, dhead].
//
// Accepted inputs follow reference src/infiniop/ops/rope/rope.h:71-205 (dtypes, 3-D or 4-D tensors,
// 1-D or 2-D position ids, contiguous tables of dhead / 2 columns, last stride 1, which strides are
// captured); the arithmetic follows src/infiniop/ops/rope/cpu/rope_cpu.cc:34-105 (see rope_device.cuh).
//
// Kernel shape: the op moves every element once in and once out (HBM-bound); a row is cut into
// 128-bit items (when all row starts are 16-byte aligned; single pairs otherwise), one per thread,
// consecutive threads on consecutive items; the table rows of a token are shared by its heads and
// stay in L1/L2.
#include "../common.h"
#include "rope_device.cuh"

namespace b200::rope {

struct Info {
    infiniDtype_t dtype, pos_dtype;
    size_t batch, seqlen, nhead, dhead, table_len, table_dim;
    ptrdiff_t y_stride_batch, y_stride_seqlen, y_stride_nhead;
    ptrdiff_t x_stride_batch, x_stride_seqlen, x_stride_nhead;
    bool pos_has_batch;
    bool gpt_j;
    bool strides_vec16; // 16-bit type, table_dim % 8 == 0 and every captured stride a multiple of 8 elements
};

struct Descriptor {
    OpDescriptorBase base;
    Info info;
};

static bool isContiguous(infiniopTensorDescriptor_t t) {
    ptrdiff_t expect = 1;
    for (size_t i = t->ndim(); i-- > 0;) {
        if (t->dim(i) != 1 && t->stride(i) != expect) {
            return false;
        }
        expect *= static_cast<ptrdiff_t>(t->dim(i));
    }
    return true;
}

static infiniStatus_t makeInfo(Info &out, infiniopTensorDescriptor_t y, infiniopTensorDescriptor_t x, infiniopTensorDescriptor_t pos,
                               infiniopTensorDescriptor_t sin, infiniopTensorDescriptor_t cos, infiniopRoPEAlgo_t algo) {
    const infiniDtype_t dtype = y->dtype;
    B200_RETURN_IF(x->dtype != dtype || sin->dtype != dtype || cos->dtype != dtype, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(dtype != INFINI_DTYPE_F16 && dtype != INFINI_DTYPE_BF16 && dtype != INFINI_DTYPE_F32 && dtype != INFINI_DTYPE_F64,
                   INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(!isIntegerDtype(pos->dtype), INFINI_STATUS_BAD_TENSOR_DTYPE);

    const bool has_batch = y->ndim() == 4;
    B200_RETURN_IF((x->ndim() == 4) != has_batch, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(!has_batch && (y->ndim() != 3 || x->ndim() != 3), INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(pos->ndim() != 1 && pos->ndim() != 2, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(sin->ndim() != 2 || cos->ndim() != 2, INFINI_STATUS_BAD_TENSOR_SHAPE);
    for (size_t i = 0; i < y->ndim(); ++i) {
        B200_RETURN_IF(y->dim(i) != x->dim(i), INFINI_STATUS_BAD_TENSOR_SHAPE);
    }
    const size_t o = has_batch ? 1 : 0;
    out.dtype = dtype;
    out.pos_dtype = pos->dtype;
    out.batch = has_batch ? y->dim(0) : 1;
    out.seqlen = y->dim(o);
    out.nhead = y->dim(o + 1);
    out.dhead = y->dim(o + 2);
    out.table_len = sin->dim(0);
    out.table_dim = sin->dim(1);
    out.pos_has_batch = pos->ndim() == 2;
    if (out.pos_has_batch) {
        B200_RETURN_IF(pos->dim(0) != out.batch || pos->dim(1) != out.seqlen, INFINI_STATUS_BAD_TENSOR_SHAPE);
    } else {
        B200_RETURN_IF(pos->dim(0) != out.seqlen, INFINI_STATUS_BAD_TENSOR_SHAPE);
    }
    B200_RETURN_IF(cos->dim(0) != out.table_len || cos->dim(1) != out.table_dim, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(out.dhead != out.table_dim * 2, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(out.dhead > 0x40000000u || out.nhead > 0x7fffffffu || out.seqlen > 0x7fffffffu || out.batch > 0x7fffffffu,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);

    B200_RETURN_IF(y->stride(o + 2) != 1 || x->stride(o + 2) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF(!isContiguous(sin) || !isContiguous(cos), INFINI_STATUS_BAD_TENSOR_STRIDES);
    // position ids are read densely (the reference indexes them as batch * seqlen + token)
    B200_RETURN_IF(!isContiguous(pos), INFINI_STATUS_BAD_TENSOR_STRIDES);

    out.y_stride_batch = has_batch ? y->stride(0) : 0;
    out.y_stride_seqlen = y->stride(o);
    out.y_stride_nhead = y->stride(o + 1);
    out.x_stride_batch = has_batch ? x->stride(0) : 0;
    out.x_stride_seqlen = x->stride(o);
    out.x_stride_nhead = x->stride(o + 1);
    out.gpt_j = algo == INFINIOP_ROPE_ALGO_GPT_J;

    const auto mult8 = [](ptrdiff_t v) { return (v % 8) == 0; };
    out.strides_vec16 = dtypeSize(dtype) == 2 && (out.table_dim % 8) == 0
                     && mult8(out.y_stride_batch) && mult8(out.y_stride_seqlen) && mult8(out.y_stride_nhead)
                     && mult8(out.x_stride_batch) && mult8(out.x_stride_seqlen) && mult8(out.x_stride_nhead);
    return INFINI_STATUS_SUCCESS;
}

struct KernelArgs {
    void *y;
    const void *x;
    const void *pos_ids;
    const void *sin_table;
    const void *cos_table;
    long long rows; // batch * seqlen * nhead
    int seqlen, nhead, table_dim;
    unsigned long long table_len;
    long long y_stride_batch, y_stride_seqlen, y_stride_nhead;
    long long x_stride_batch, x_stride_seqlen, x_stride_nhead;
    int pos_dtype;
    int pos_has_batch;
    int vec;
    int small; // rows * items per row (rounded up to whole blocks) fits 32 bits
};

constexpr int kThreads = 256;

// One thread per item (see rotateItem); consecutive threads take consecutive items of a row, then the next row.
template <typename T, bool kGptJ>
__global__ void __launch_bounds__(kThreads) ropeRowsKernel(const KernelArgs a) {
    const int per_row = itemsPerRow<kGptJ>(a.table_dim, a.vec != 0);
    long long row, head, tok, b;
    int item;
    if (a.small) {
        // fewer than 2^32 items: 32-bit divisions (a 64-bit one costs several times as much)
        const unsigned idx = blockIdx.x * static_cast<unsigned>(kThreads) + threadIdx.x;
        const unsigned r = idx / static_cast<unsigned>(per_row);
        const unsigned th = r / static_cast<unsigned>(a.nhead);
        item = static_cast<int>(idx - r * per_row);
        row = r;
        head = r - th * a.nhead;
        b = th / static_cast<unsigned>(a.seqlen);
        tok = th - static_cast<unsigned>(b) * a.seqlen;
    } else {
        const long long idx = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
        row = idx / per_row;
        item = static_cast<int>(idx - row * per_row);
        head = row % a.nhead;
        tok = (row / a.nhead) % a.seqlen;
        b = row / (static_cast<long long>(a.nhead) * a.seqlen);
    }
    if (row >= a.rows) {
        return;
    }
    const unsigned long long pos = loadPosition(a.pos_ids, (a.pos_has_batch ? b * a.seqlen : 0) + tok, a.pos_dtype);
    const T *x = static_cast<const T *>(a.x) + b * a.x_stride_batch + tok * a.x_stride_seqlen + head * a.x_stride_nhead;
    T *y = static_cast<T *>(a.y) + b * a.y_stride_batch + tok * a.y_stride_seqlen + head * a.y_stride_nhead;
    const bool in_table = pos < a.table_len;
    const T *sin_row = in_table ? static_cast<const T *>(a.sin_table) + pos * a.table_dim : nullptr;
    const T *cos_row = in_table ? static_cast<const T *>(a.cos_table) + pos * a.table_dim : nullptr;
    rotateItem<T, kGptJ>(y, x, sin_row, cos_row, a.table_dim, item, a.vec != 0);
}

// Vector path, two rows per thread (row r and row r + ceil(rows / 2), the same item of each): the position
// ids of both are loaded first, then the x words of both, then the table words of both, so that twice the
// bytes are in flight while a thread waits.  16-bit types and 32-bit item counts only.
template <typename T, bool kGptJ>
__global__ void __launch_bounds__(kThreads) ropeRowPairsKernel(const KernelArgs a) {
    const unsigned per_row = static_cast<unsigned>(itemsPerRow<kGptJ>(a.table_dim, true));
    const unsigned half_rows = static_cast<unsigned>((a.rows + 1) / 2);
    const unsigned idx = blockIdx.x * static_cast<unsigned>(kThreads) + threadIdx.x;
    const unsigned r0 = idx / per_row;
    if (r0 >= half_rows) {
        return;
    }
    const int item = static_cast<int>(idx - r0 * per_row);
    const T *x[2];
    T *y[2];
    const T *sin_row[2], *cos_row[2];
    bool live[2];
    unsigned long long pos[2];
    long long pos_index[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const unsigned r = r0 + u * half_rows;
        live[u] = r < a.rows;
        const unsigned th = r / static_cast<unsigned>(a.nhead);
        const unsigned head = r - th * a.nhead;
        const unsigned b = th / static_cast<unsigned>(a.seqlen);
        const unsigned tok = th - b * a.seqlen;
        pos_index[u] = (a.pos_has_batch ? static_cast<long long>(b) * a.seqlen : 0) + tok;
        x[u] = static_cast<const T *>(a.x) + b * a.x_stride_batch + tok * a.x_stride_seqlen + head * a.x_stride_nhead;
        y[u] = static_cast<T *>(a.y) + b * a.y_stride_batch + tok * a.y_stride_seqlen + head * a.y_stride_nhead;
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        pos[u] = live[u] ? loadPosition(a.pos_ids, pos_index[u], a.pos_dtype) : ~0ull;
    }
    VecItem<T> in[2];
    VecTables<T> t[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        if (live[u]) {
            loadItemVec<T, kGptJ>(in[u], x[u], a.table_dim, item);
        }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const bool in_table = pos[u] < a.table_len;
        sin_row[u] = in_table ? static_cast<const T *>(a.sin_table) + pos[u] * a.table_dim : nullptr;
        cos_row[u] = in_table ? static_cast<const T *>(a.cos_table) + pos[u] * a.table_dim : nullptr;
        if (live[u]) {
            loadTablesVec<T, kGptJ>(t[u], sin_row[u], cos_row[u], item);
        }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        if (live[u]) {
            rotateStoreVec<T, kGptJ>(y[u], in[u], t[u], sin_row[u] != nullptr, a.table_dim, item);
        }
    }
}

template <typename T>
static infiniStatus_t launch(const Info &I, const KernelArgs &a, cudaStream_t stream) {
    if constexpr (sizeof(T) == 2) {
        const long long per_row_vec = I.gpt_j ? itemsPerRow<true>(a.table_dim, true) : itemsPerRow<false>(a.table_dim, true);
        const long long pair_blocks = ((a.rows + 1) / 2 * per_row_vec + kThreads - 1) / kThreads;
        // rows of the two halves must not overlap in y (they cannot for a tensor that does not alias itself)
        if (a.vec != 0 && a.rows >= 2 && a.rows <= 0x7fffffffLL && pair_blocks * kThreads <= 0x7fffffffLL) {
            if (I.gpt_j) {
                ropeRowPairsKernel<T, true><<<static_cast<unsigned>(pair_blocks), kThreads, 0, stream>>>(a);
            } else {
                ropeRowPairsKernel<T, false><<<static_cast<unsigned>(pair_blocks), kThreads, 0, stream>>>(a);
            }
            return checkLaunch("ropeRowPairsKernel");
        }
    }
    const long long per_row = I.gpt_j ? itemsPerRow<true>(a.table_dim, a.vec != 0) : itemsPerRow<false>(a.table_dim, a.vec != 0);
    const long long blocks = (a.rows * per_row + kThreads - 1) / kThreads;
    B200_RETURN_IF(blocks > 0x7fffffffLL, INFINI_STATUS_BAD_TENSOR_SHAPE);
    KernelArgs args = a;
    args.small = blocks * kThreads <= 0xffffffffLL ? 1 : 0;
    if (I.gpt_j) {
        ropeRowsKernel<T, true><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(args);
    } else {
        ropeRowsKernel<T, false><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(args);
    }
    return checkLaunch("ropeRowsKernel");
}

} // namespace b200::rope

using b200::rope::Descriptor;

__INFINI_C infiniStatus_t infiniopCreateRoPEDescriptor(
    infiniopHandle_t handle,
    infiniopRoPEDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t y,
    infiniopTensorDescriptor_t x,
    infiniopTensorDescriptor_t pos_ids,
    infiniopTensorDescriptor_t sin_table,
    infiniopTensorDescriptor_t cos_table,
    infiniopRoPEAlgo_t algo) {
    B200_RETURN_IF(handle == nullptr || desc_ptr == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(y == nullptr || x == nullptr || pos_ids == nullptr || sin_table == nullptr || cos_table == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    // the reference reports an algorithm outside the enum with the same status (rope.h:79-81)
    B200_RETURN_IF(static_cast<int>(algo) < 0 || static_cast<int>(algo) >= INFINIOP_ROPE_ALGO_COUNT, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(handle->device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);

    b200::rope::Info info;
    const infiniStatus_t st = b200::rope::makeInfo(info, y, x, pos_ids, sin_table, cos_table, algo);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    auto *h = reinterpret_cast<b200::Handle *>(handle);
    auto *d = new Descriptor{{handle->device, handle->device_id, b200::OpKind::RoPE, h->props}, info};
    *desc_ptr = reinterpret_cast<infiniopRoPEDescriptor_t>(d);
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopGetRoPEWorkspaceSize(infiniopRoPEDescriptor_t desc, size_t *size) {
    B200_RETURN_IF(desc == nullptr || size == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(reinterpret_cast<Descriptor *>(desc)->base.kind != b200::OpKind::RoPE, INFINI_STATUS_BAD_PARAM);
    *size = 0;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopRoPE(
    infiniopRoPEDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *y,
    const void *x,
    void const *pos_ids,
    void const *sin_table,
    void const *cos_table,
    void *stream) {
    (void)workspace;
    (void)workspace_size;
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<Descriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::RoPE, INFINI_STATUS_BAD_PARAM);
    const auto &I = d->info;
    const long long rows = static_cast<long long>(I.batch) * static_cast<long long>(I.seqlen) * static_cast<long long>(I.nhead);
    if (rows == 0 || I.dhead == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    B200_RETURN_IF(y == nullptr || x == nullptr || pos_ids == nullptr || sin_table == nullptr || cos_table == nullptr,
                   INFINI_STATUS_NULL_POINTER);

    const auto addr = [](const void *p) { return reinterpret_cast<uintptr_t>(p); };
    b200::rope::KernelArgs a{};
    a.y = y;
    a.x = x;
    a.pos_ids = pos_ids;
    a.sin_table = sin_table;
    a.cos_table = cos_table;
    a.rows = rows;
    a.seqlen = static_cast<int>(I.seqlen);
    a.nhead = static_cast<int>(I.nhead);
    a.table_dim = static_cast<int>(I.table_dim);
    a.table_len = I.table_len;
    a.y_stride_batch = I.y_stride_batch;
    a.y_stride_seqlen = I.y_stride_seqlen;
    a.y_stride_nhead = I.y_stride_nhead;
    a.x_stride_batch = I.x_stride_batch;
    a.x_stride_seqlen = I.x_stride_seqlen;
    a.x_stride_nhead = I.x_stride_nhead;
    a.pos_dtype = static_cast<int>(I.pos_dtype);
    a.pos_has_batch = I.pos_has_batch ? 1 : 0;
    a.vec = I.strides_vec16 && ((addr(y) | addr(x) | addr(sin_table) | addr(cos_table)) & 15u) == 0;

    auto cuda_stream = static_cast<cudaStream_t>(stream);
    switch (I.dtype) {
    case INFINI_DTYPE_F16:
        return b200::rope::launch<__half>(I, a, cuda_stream);
    case INFINI_DTYPE_BF16:
        return b200::rope::launch<__nv_bfloat16>(I, a, cuda_stream);
    case INFINI_DTYPE_F32:
        return b200::rope::launch<float>(I, a, cuda_stream);
    default:
        return b200::rope::launch<double>(I, a, cuda_stream);
    }
}

__INFINI_C infiniStatus_t infiniopDestroyRoPEDescriptor(infiniopRoPEDescriptor_t desc) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<Descriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::RoPE, INFINI_STATUS_BAD_PARAM);
    delete d;
    return INFINI_STATUS_SUCCESS;
}
