// infiniopPagedDecodeStep: append the newest K/V row of every sequence, then attend - the work of
// infiniopPagedCaching + infiniopPagedAttention for one decode layer behind one entry point.
//
// The reference has no such operator (its callers issue the two separately:
// src/infinicore/ops/paged_caching/paged_caching_infiniop.cc:38-51 then
// src/infinicore/ops/paged_attention/paged_attention_infiniop.cc:47-64).  When the streaming kernel
// takes the problem, the append rides inside it: the warp that reaches a sequence's last tile swaps
// the new row into its staged copy and stores it into the cache, so no separate launch is needed
// and no other CTA has to see the cache write.  Otherwise a small append kernel runs first and the
// generic attention kernel follows in stream order.
//
// The RoPE form (infiniopPagedDecodeStepRoPE) also does the work of the two infiniopRoPE calls a
// decode layer issues on q and on the new K before it caches and attends: one small kernel writes
// the rotated q and K rows into the workspace, and the attention kernels take q and the appended
// K row from there.  q and new_k themselves stay as they were.
#include "kernels.h"

#include "../rope/rope_device.cuh"

#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstring>

namespace b200::paged_attention {

namespace {

struct StepDescriptor {
    OpDescriptorBase base;
    Info info;
    StreamPlan stream;
    size_t workspace_bytes;
    ptrdiff_t new_k_seq_stride, new_v_seq_stride;
    bool rows_vectorisable; // row starts stay 16-byte aligned given aligned bases
    int fuse_mode = -1; // INFINIOP_PAGED_DECODE_STEP_FUSE: 1 always hand the rows to the attention kernel, 0 never, unset: by batch size
    // RoPE form only
    bool has_rope = false;
    bool gpt_j = false;
    infiniDtype_t pos_dtype = INFINI_DTYPE_I64;
    size_t table_len = 0;
    ptrdiff_t q_seq_stride = 0, q_head_stride = 0; // of the caller's q (Info holds the dense strides of the rotated copy)
    size_t attention_workspace_bytes = 0;          // rounded up to 256: the rotated q starts here
    size_t rotated_q_bytes = 0;                    // rounded up to 256: the rotated K rows follow
};

struct RopeRowsArgs {
    void *q_rot;       // [num_seqs, num_heads, head_size] dense
    void *k_rot;       // [num_seqs, num_kv_heads, head_size] dense
    const void *q;
    const void *new_k;
    const void *pos_ids;
    const void *sin_table;
    const void *cos_table;
    int num_seqs, num_heads, num_kv_heads, head_size;
    long long q_seq_stride, q_head_stride, new_k_seq_stride;
    unsigned long long table_len;
    int pos_dtype;
    int vec;
};

// One thread per item of a (sequence, q-head | kv-head) row (see rotateItem): rotate it by the sequence's position id.
template <typename T, bool kGptJ>
__global__ void __launch_bounds__(128) pagedRopeRowsKernel(const RopeRowsArgs a) {
    // Programmatic dependent launch on both sides.  This kernel may itself have started under the tail of
    // its predecessor in the stream: it touches no global memory before the wait returns (predecessor complete,
    // its writes visible).  The attention kernel that follows is launched the same way: let its CTAs become
    // resident and run their shared-memory prologue now; it reads nothing from global memory before its own
    // wait, which returns only when this whole grid has finished and its rows are visible.  Every CTA waits
    // before it exits, so the ordering is transitive.  Both instructions are no-ops for a plain launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int table_dim = a.head_size / 2;
    const int per_row = b200::rope::itemsPerRow<kGptJ>(table_dim, a.vec != 0);
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int rows_per_seq = a.num_heads + a.num_kv_heads;
    const long long row = idx / per_row;
    if (row >= static_cast<long long>(a.num_seqs) * rows_per_seq) {
        return;
    }
    const int item = static_cast<int>(idx - row * per_row);
    const int seq = static_cast<int>(row / rows_per_seq);
    const int h = static_cast<int>(row % rows_per_seq);
    const T *src;
    T *dst;
    if (h < a.num_heads) {
        src = static_cast<const T *>(a.q) + seq * a.q_seq_stride + h * a.q_head_stride;
        dst = static_cast<T *>(a.q_rot) + (static_cast<long long>(seq) * a.num_heads + h) * a.head_size;
    } else {
        const int kv = h - a.num_heads;
        src = static_cast<const T *>(a.new_k) + seq * a.new_k_seq_stride + static_cast<long long>(kv) * a.head_size;
        dst = static_cast<T *>(a.k_rot) + (static_cast<long long>(seq) * a.num_kv_heads + kv) * a.head_size;
    }
    const unsigned long long pos = b200::rope::loadPosition(a.pos_ids, seq, a.pos_dtype);
    const bool in_table = pos < a.table_len;
    const T *sin_row = in_table ? static_cast<const T *>(a.sin_table) + pos * table_dim : nullptr;
    const T *cos_row = in_table ? static_cast<const T *>(a.cos_table) + pos * table_dim : nullptr;
    b200::rope::rotateItem<T, kGptJ>(dst, src, sin_row, cos_row, table_dim, item, a.vec != 0);
}

template <typename T>
infiniStatus_t launchRopeRows(const RopeRowsArgs &a, bool gpt_j, bool use_pdl, cudaStream_t stream) {
    const long long rows = static_cast<long long>(a.num_seqs) * (a.num_heads + a.num_kv_heads);
    const int table_dim = a.head_size / 2;
    const long long per_row = gpt_j ? b200::rope::itemsPerRow<true>(table_dim, a.vec != 0) : b200::rope::itemsPerRow<false>(table_dim, a.vec != 0);
    const unsigned blocks = static_cast<unsigned>((rows * per_row + 127) / 128);
    if (blocks == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    cudaLaunchAttribute pdl;
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl.val.programmaticStreamSerializationAllowed = use_pdl ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cfg.attrs = &pdl;
    cfg.numAttrs = 1;
    const cudaError_t err = gpt_j ? cudaLaunchKernelEx(&cfg, pagedRopeRowsKernel<T, true>, a)
                                  : cudaLaunchKernelEx(&cfg, pagedRopeRowsKernel<T, false>, a);
    (void)err; // reported through cudaGetLastError below
    return checkLaunch("pagedRopeRowsKernel");
}

// One warp per (sequence, kv-head, K | V) row.
template <typename T>
__global__ void __launch_bounds__(128) pagedAppendRowsKernel(const DecodeParams p, int vec_ok) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int rows = p.num_seqs * p.num_kv_heads * 2;
    if (warp >= rows) {
        return;
    }
    const int is_v = warp & 1;
    const int kv_head = (warp >> 1) % p.num_kv_heads;
    const int seq = (warp >> 1) / p.num_kv_heads;
    long long len = loadIndex(p.seq_lens, seq, p.index_is_64);
    const long long capacity = static_cast<long long>(p.max_blocks_per_seq) * p.block_size;
    len = len > capacity ? capacity : len;
    if (len <= 0) {
        return;
    }
    const long long n = len - 1;
    const long long block = loadIndex(p.block_tables, seq * p.bt_seq_stride + n / p.block_size, p.index_is_64);
    if (static_cast<unsigned long long>(block) >= static_cast<unsigned long long>(p.num_blocks)) {
        // a table entry outside the pool: nothing is stored (reported when index checking is on)
        if (lane == 0 && p.check_indices) {
            atomicOr(p.kernel_flags, 2u);
        }
        return;
    }
    const int row = static_cast<int>(n % p.block_size);
    const int width = is_v ? p.value_size : p.head_size;
    const T *src = is_v ? static_cast<const T *>(p.new_v) + seq * p.new_v_seq_stride + kv_head * p.value_size
                        : static_cast<const T *>(p.new_k) + seq * p.new_k_seq_stride + kv_head * p.head_size;
    T *dst = is_v ? static_cast<T *>(const_cast<void *>(p.v_cache)) + block * p.v_block_stride + kv_head * p.v_head_stride + row * p.v_row_stride
                  : static_cast<T *>(const_cast<void *>(p.k_cache)) + block * p.k_block_stride + kv_head * p.k_head_stride + row * p.k_row_stride;
    if (vec_ok) {
        for (int i = lane * 8; i < width; i += 256) {
            *reinterpret_cast<uint4 *>(dst + i) = *reinterpret_cast<const uint4 *>(src + i);
        }
    } else {
        for (int i = lane; i < width; i += 32) {
            dst[i] = src[i];
        }
    }
}

} // namespace

infiniStatus_t launchAppendNewRows(const Info &info, const DecodeParams &p, cudaStream_t stream) {
    const long long rows = static_cast<long long>(p.num_seqs) * p.num_kv_heads * 2;
    if (rows == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    const auto addr = [](const void *ptr) { return reinterpret_cast<uintptr_t>(ptr); };
    const auto mult8 = [](long long v) { return (v % 8) == 0; };
    const int vec_ok = ((addr(p.k_cache) | addr(p.v_cache) | addr(p.new_k) | addr(p.new_v)) & 15u) == 0 && mult8(p.head_size) && mult8(p.value_size)
                       && mult8(p.new_k_seq_stride) && mult8(p.new_v_seq_stride) && mult8(p.k_block_stride) && mult8(p.k_head_stride)
                       && mult8(p.k_row_stride) && mult8(p.v_block_stride) && mult8(p.v_head_stride) && mult8(p.v_row_stride);
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 127) / 128);
    if (info.dtype == INFINI_DTYPE_F16) {
        pagedAppendRowsKernel<__half><<<blocks, 128, 0, stream>>>(p, vec_ok);
    } else {
        pagedAppendRowsKernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(p, vec_ok);
    }
    return checkLaunch("pagedAppendRowsKernel");
}

// defined in operator.cu
DecodeParams makeDecodeParams(const Info &I, void *out, const void *q, const void *k_cache, const void *v_cache,
                              const void *block_tables, const void *seq_lens, const void *alibi_slopes);

} // namespace b200::paged_attention

using b200::paged_attention::StepDescriptor;

namespace {

constexpr size_t roundUp256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

bool denseTable(infiniopTensorDescriptor_t t) {
    return t->ndim() == 2 && (t->dim(1) == 1 || t->stride(1) == 1) && (t->dim(0) == 1 || t->stride(0) == static_cast<ptrdiff_t>(t->dim(1)));
}

// Shared by both forms; the three RoPE descriptors are null for the plain one.
infiniStatus_t createStep(
    infiniopHandle_t handle,
    infiniopPagedDecodeStepDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t new_k_desc,
    infiniopTensorDescriptor_t new_v_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    infiniopTensorDescriptor_t pos_ids_desc,
    infiniopTensorDescriptor_t sin_desc,
    infiniopTensorDescriptor_t cos_desc,
    infiniopRoPEAlgo_t algo,
    float scale) {
    const bool rope = pos_ids_desc != nullptr;
    B200_RETURN_IF(handle == nullptr || desc_ptr == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(out_desc == nullptr || q_desc == nullptr || k_cache_desc == nullptr || v_cache_desc == nullptr
                       || new_k_desc == nullptr || new_v_desc == nullptr || block_tables_desc == nullptr || seq_lens_desc == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(handle->device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);

    b200::paged_attention::Info info;
    infiniStatus_t st = b200::paged_attention::makeInfo(info, out_desc, q_desc, k_cache_desc, v_cache_desc,
                                                        block_tables_desc, seq_lens_desc, alibi_slopes_desc, scale);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    B200_RETURN_IF(info.num_seqs > 0x7fffffffu || info.num_heads > 65535u || info.max_num_blocks_per_seq > 0x7fffffffu
                       || info.block_size > 65536u || info.num_blocks > 0x7fffffffu,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    // the new rows: one token per sequence, the cache's dtype, dense heads
    B200_RETURN_IF(new_k_desc->dtype != info.dtype || new_v_desc->dtype != info.dtype, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(new_k_desc->ndim() != 3 || new_v_desc->ndim() != 3, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(new_k_desc->dim(0) != info.num_seqs || new_k_desc->dim(1) != info.num_kv_heads || new_k_desc->dim(2) != info.head_size,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(new_v_desc->dim(0) != info.num_seqs || new_v_desc->dim(1) != info.num_kv_heads || new_v_desc->dim(2) != info.value_size,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(new_k_desc->stride(2) != 1 || new_v_desc->stride(2) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF(new_k_desc->stride(1) != static_cast<ptrdiff_t>(info.head_size)
                       || new_v_desc->stride(1) != static_cast<ptrdiff_t>(info.value_size),
                   INFINI_STATUS_BAD_TENSOR_STRIDES);

    auto *h = reinterpret_cast<b200::Handle *>(handle);
    auto d = std::make_unique<StepDescriptor>();
    d->base = {handle->device, handle->device_id, b200::OpKind::PagedDecodeStep, h->props};
    d->new_k_seq_stride = new_k_desc->stride(0);
    d->new_v_seq_stride = new_v_desc->stride(0);
    d->rows_vectorisable = (d->new_k_seq_stride % 8) == 0 && (d->new_v_seq_stride % 8) == 0;

    if (rope) {
        // position ids [num_seqs] of any integer type; tables [table_len, head_size / 2] of the data type
        // (the checks of infiniopCreateRoPEDescriptor for x = q viewed as [num_seqs, num_heads, head_size])
        B200_RETURN_IF(sin_desc == nullptr || cos_desc == nullptr, INFINI_STATUS_NULL_POINTER);
        B200_RETURN_IF(static_cast<int>(algo) < 0 || static_cast<int>(algo) >= INFINIOP_ROPE_ALGO_COUNT, INFINI_STATUS_NULL_POINTER);
        B200_RETURN_IF(sin_desc->dtype != info.dtype || cos_desc->dtype != info.dtype, INFINI_STATUS_BAD_TENSOR_DTYPE);
        B200_RETURN_IF(!b200::rope::isIntegerDtype(pos_ids_desc->dtype), INFINI_STATUS_BAD_TENSOR_DTYPE);
        B200_RETURN_IF(pos_ids_desc->ndim() != 1 || pos_ids_desc->dim(0) != info.num_seqs, INFINI_STATUS_BAD_TENSOR_SHAPE);
        B200_RETURN_IF(sin_desc->ndim() != 2 || cos_desc->ndim() != 2, INFINI_STATUS_BAD_TENSOR_SHAPE);
        B200_RETURN_IF(sin_desc->dim(0) != cos_desc->dim(0) || sin_desc->dim(1) != cos_desc->dim(1), INFINI_STATUS_BAD_TENSOR_SHAPE);
        B200_RETURN_IF(sin_desc->dim(1) * 2 != info.head_size, INFINI_STATUS_BAD_TENSOR_SHAPE);
        B200_RETURN_IF(info.num_seqs > 1 && pos_ids_desc->stride(0) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
        B200_RETURN_IF(!denseTable(sin_desc) || !denseTable(cos_desc), INFINI_STATUS_BAD_TENSOR_STRIDES);
        d->has_rope = true;
        d->gpt_j = algo == INFINIOP_ROPE_ALGO_GPT_J;
        d->pos_dtype = pos_ids_desc->dtype;
        d->table_len = sin_desc->dim(0);
        d->q_seq_stride = info.q_seq_stride;
        d->q_head_stride = info.q_head_stride;
        // the attention kernels read the rotated copy, which is dense
        info.q_seq_stride = static_cast<ptrdiff_t>(info.num_heads * info.head_size);
        info.q_head_stride = static_cast<ptrdiff_t>(info.head_size);
    }
    d->info = info;
    d->info.kernel_flags = h->props->kernel_flags;
    d->info.check_indices = b200::paged_attention::checkIndicesFromEnv();

    // the same path selection as infiniopPagedAttention (INFINIOP_PAGED_DECODE_PATH = auto | stream | generic)
    const char *path = std::getenv("INFINIOP_PAGED_DECODE_PATH");
    const bool force_generic = (path != nullptr) && std::strcmp(path, "generic") == 0;
    if (!force_generic) {
        d->stream = b200::paged_attention::planStream(info, *h->props);
    }
    if (path != nullptr && std::strcmp(path, "stream") == 0 && !d->stream.eligible) {
        std::fprintf(stderr, "[infiniop] INFINIOP_PAGED_DECODE_PATH=stream but this problem is not eligible for the streaming kernel\n");
        return INFINI_STATUS_BAD_PARAM;
    }
    d->workspace_bytes = d->stream.eligible ? d->stream.workspace_bytes : 0;
    if (const char *fuse = std::getenv("INFINIOP_PAGED_DECODE_STEP_FUSE")) {
        d->fuse_mode = std::strcmp(fuse, "1") == 0 ? 1 : (std::strcmp(fuse, "0") == 0 ? 0 : -1);
    }
    if (rope) {
        const size_t elem = b200::dtypeSize(info.dtype);
        d->attention_workspace_bytes = roundUp256(d->workspace_bytes);
        d->rotated_q_bytes = roundUp256(info.num_seqs * info.num_heads * info.head_size * elem);
        d->workspace_bytes = d->attention_workspace_bytes + d->rotated_q_bytes + roundUp256(info.num_seqs * info.num_kv_heads * info.head_size * elem);
    }
    *desc_ptr = reinterpret_cast<infiniopPagedDecodeStepDescriptor_t>(d.release());
    return INFINI_STATUS_SUCCESS;
}

infiniStatus_t runStep(
    StepDescriptor *d,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    void *k_cache,
    void *v_cache,
    const void *new_k,
    const void *new_v,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    const void *pos_ids,
    const void *sin_table,
    const void *cos_table,
    void *stream) {
    const auto &I = d->info;
    if (I.num_seqs == 0 || I.num_heads == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    B200_RETURN_IF(out == nullptr || q == nullptr || k_cache == nullptr || v_cache == nullptr || new_k == nullptr || new_v == nullptr
                       || block_tables == nullptr || seq_lens == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(I.has_alibi && alibi_slopes == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(d->has_rope && (pos_ids == nullptr || sin_table == nullptr || cos_table == nullptr), INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(workspace_size < d->workspace_bytes, INFINI_STATUS_INSUFFICIENT_WORKSPACE);
    B200_RETURN_IF(d->workspace_bytes > 0 && workspace == nullptr, INFINI_STATUS_NULL_POINTER);

    auto cuda_stream = static_cast<cudaStream_t>(stream);
    const auto addr = [](const void *ptr) { return reinterpret_cast<uintptr_t>(ptr); };
    long long new_k_seq_stride = d->new_k_seq_stride;
    if (d->has_rope) {
        // rotated q and K rows go to the tail of the workspace; from here on they ARE q and new_k
        B200_RETURN_IF((addr(workspace) & 255u) != 0, INFINI_STATUS_BAD_PARAM);
        auto *bytes = static_cast<unsigned char *>(workspace);
        b200::paged_attention::RopeRowsArgs r{};
        r.q_rot = bytes + d->attention_workspace_bytes;
        r.k_rot = bytes + d->attention_workspace_bytes + d->rotated_q_bytes;
        r.q = q;
        r.new_k = new_k;
        r.pos_ids = pos_ids;
        r.sin_table = sin_table;
        r.cos_table = cos_table;
        r.num_seqs = static_cast<int>(I.num_seqs);
        r.num_heads = static_cast<int>(I.num_heads);
        r.num_kv_heads = static_cast<int>(I.num_kv_heads);
        r.head_size = static_cast<int>(I.head_size);
        r.q_seq_stride = d->q_seq_stride;
        r.q_head_stride = d->q_head_stride;
        r.new_k_seq_stride = d->new_k_seq_stride;
        r.table_len = d->table_len;
        r.pos_dtype = static_cast<int>(d->pos_dtype);
        r.vec = (I.head_size % 16) == 0 && (d->q_seq_stride % 8) == 0 && (d->q_head_stride % 8) == 0 && (d->new_k_seq_stride % 8) == 0
             && ((addr(q) | addr(new_k) | addr(sin_table) | addr(cos_table)) & 15u) == 0;
        // only in front of the streaming kernels, which wait for their predecessor themselves
        const bool use_pdl = d->stream.eligible && d->stream.use_pdl;
        const infiniStatus_t st = I.dtype == INFINI_DTYPE_F16
                                    ? b200::paged_attention::launchRopeRows<__half>(r, d->gpt_j, use_pdl, cuda_stream)
                                    : b200::paged_attention::launchRopeRows<__nv_bfloat16>(r, d->gpt_j, use_pdl, cuda_stream);
        B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
        q = r.q_rot;
        new_k = r.k_rot;
        new_k_seq_stride = static_cast<long long>(I.num_kv_heads * I.head_size);
    }

    auto p = b200::paged_attention::makeDecodeParams(I, out, q, k_cache, v_cache, block_tables, seq_lens, alibi_slopes);
    p.new_k = new_k;
    p.new_v = new_v;
    p.new_k_seq_stride = new_k_seq_stride;
    p.new_v_seq_stride = d->new_v_seq_stride;
    const bool rows_vectorisable = (new_k_seq_stride % 8) == 0 && (d->new_v_seq_stride % 8) == 0;
    // The row hand-over costs a worker one dependent round trip to global memory at the end of every unit
    // (sequence, kv-head, head tile).  With at most one unit per worker on average that is cheaper than a
    // launch; with several it piles up (256 ragged sequences: 0.786 ms against 0.735 ms for append kernel +
    // attention), so larger batches take the append kernel.  INFINIOP_PAGED_DECODE_STEP_FUSE = 1 | 0 overrides.
    const size_t units = I.num_seqs * I.num_kv_heads * static_cast<size_t>(d->stream.head_tiles_per_group);
    const bool wanted = d->fuse_mode == 1 || (d->fuse_mode < 0 && units <= static_cast<size_t>(d->stream.num_workers));
    const bool fused = wanted && d->stream.eligible && b200::paged_attention::streamTakesPointers(d->stream, p, workspace)
                       && rows_vectorisable && ((addr(new_k) | addr(new_v)) & 15u) == 0;
    if (fused) {
        return b200::paged_attention::launchDecodeStream(I, d->stream, p, workspace, workspace_size, cuda_stream);
    }
    // append first, then the attention kernels without the row hand-over
    const infiniStatus_t st = b200::paged_attention::launchAppendNewRows(I, p, cuda_stream);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    p.new_k = nullptr;
    p.new_v = nullptr;
    if (d->stream.eligible) {
        return b200::paged_attention::launchDecodeStream(I, d->stream, p, workspace, workspace_size, cuda_stream);
    }
    return b200::paged_attention::launchDecodeGeneric(I, p, cuda_stream);
}

} // namespace

__INFINI_C infiniStatus_t infiniopCreatePagedDecodeStepDescriptor(
    infiniopHandle_t handle,
    infiniopPagedDecodeStepDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t new_k_desc,
    infiniopTensorDescriptor_t new_v_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    float scale) {
    return createStep(handle, desc_ptr, out_desc, q_desc, k_cache_desc, v_cache_desc, new_k_desc, new_v_desc, block_tables_desc,
                      seq_lens_desc, alibi_slopes_desc, nullptr, nullptr, nullptr, INFINIOP_ROPE_ALGO_GPT_NEOX, scale);
}

__INFINI_C infiniStatus_t infiniopCreatePagedDecodeStepRoPEDescriptor(
    infiniopHandle_t handle,
    infiniopPagedDecodeStepDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t new_k_desc,
    infiniopTensorDescriptor_t new_v_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    infiniopTensorDescriptor_t pos_ids_desc,
    infiniopTensorDescriptor_t sin_table_desc,
    infiniopTensorDescriptor_t cos_table_desc,
    infiniopRoPEAlgo_t algo,
    float scale) {
    B200_RETURN_IF(pos_ids_desc == nullptr || sin_table_desc == nullptr || cos_table_desc == nullptr, INFINI_STATUS_NULL_POINTER);
    return createStep(handle, desc_ptr, out_desc, q_desc, k_cache_desc, v_cache_desc, new_k_desc, new_v_desc, block_tables_desc,
                      seq_lens_desc, alibi_slopes_desc, pos_ids_desc, sin_table_desc, cos_table_desc, algo, scale);
}

__INFINI_C infiniStatus_t infiniopGetPagedDecodeStepWorkspaceSize(infiniopPagedDecodeStepDescriptor_t desc, size_t *size) {
    B200_RETURN_IF(desc == nullptr || size == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<StepDescriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::PagedDecodeStep, INFINI_STATUS_BAD_PARAM);
    *size = d->workspace_bytes;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopPagedDecodeStep(
    infiniopPagedDecodeStepDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    void *k_cache,
    void *v_cache,
    const void *new_k,
    const void *new_v,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    void *stream) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<StepDescriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::PagedDecodeStep || d->has_rope, INFINI_STATUS_BAD_PARAM);
    return runStep(d, workspace, workspace_size, out, q, k_cache, v_cache, new_k, new_v, block_tables, seq_lens, alibi_slopes,
                   nullptr, nullptr, nullptr, stream);
}

__INFINI_C infiniStatus_t infiniopPagedDecodeStepRoPE(
    infiniopPagedDecodeStepDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    void *k_cache,
    void *v_cache,
    const void *new_k,
    const void *new_v,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    const void *pos_ids,
    const void *sin_table,
    const void *cos_table,
    void *stream) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<StepDescriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::PagedDecodeStep || !d->has_rope, INFINI_STATUS_BAD_PARAM);
    return runStep(d, workspace, workspace_size, out, q, k_cache, v_cache, new_k, new_v, block_tables, seq_lens, alibi_slopes,
                   pos_ids, sin_table, cos_table, stream);
}

__INFINI_C infiniStatus_t infiniopDestroyPagedDecodeStepDescriptor(infiniopPagedDecodeStepDescriptor_t desc) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<StepDescriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::PagedDecodeStep, INFINI_STATUS_BAD_PARAM);
    delete d;
    return INFINI_STATUS_SUCCESS;
}
