// C entry points of infiniopPagedAttention and the descriptor behind them.
//
// Replaces reference src/infiniop/ops/paged_attention/operator.cc:21-190 and
// nvidia/paged_attention_nvidia.cu:182-443.  Differences a caller can observe:
//  * the workspace size is this library's own (callers query it; the reference's
//    8 * seqs * heads * (value + 2) * 4 formula is not part of the contract);
//  * tuning knobs are read from the environment once, when the descriptor is created,
//    never on the execute path;
//  * a failed kernel launch is reported as INFINI_STATUS_INTERNAL_ERROR.
#include "kernels.h"

#include <cstdlib>
#include <cstring>

namespace b200::paged_attention {

struct Descriptor {
    OpDescriptorBase base;
    Info info;
    StreamPlan stream;
    size_t workspace_bytes;
};

DecodeParams makeDecodeParams(const Info &I, void *out, const void *q, const void *k_cache, const void *v_cache,
                              const void *block_tables, const void *seq_lens, const void *alibi_slopes) {
    DecodeParams p;
    p.out = out;
    p.q = q;
    p.k_cache = k_cache;
    p.v_cache = v_cache;
    p.block_tables = block_tables;
    p.seq_lens = seq_lens;
    p.alibi_slopes = I.has_alibi ? static_cast<const float *>(alibi_slopes) : nullptr;
    p.num_seqs = static_cast<int>(I.num_seqs);
    p.num_heads = static_cast<int>(I.num_heads);
    p.num_kv_heads = static_cast<int>(I.num_kv_heads);
    p.group_size = static_cast<int>(I.num_heads / I.num_kv_heads);
    p.head_size = static_cast<int>(I.head_size);
    p.value_size = static_cast<int>(I.value_size);
    p.block_size = static_cast<int>(I.block_size);
    p.max_blocks_per_seq = static_cast<int>(I.max_num_blocks_per_seq);
    p.index_is_64 = (I.index_dtype == INFINI_DTYPE_I64) ? 1 : 0;
    p.q_seq_stride = I.q_seq_stride;
    p.q_head_stride = I.q_head_stride;
    p.o_seq_stride = I.o_seq_stride;
    p.o_head_stride = I.o_head_stride;
    p.k_block_stride = I.k_block_stride;
    p.k_head_stride = I.k_head_stride;
    p.k_row_stride = I.k_row_stride;
    p.v_block_stride = I.v_block_stride;
    p.v_head_stride = I.v_head_stride;
    p.v_row_stride = I.v_row_stride;
    p.bt_seq_stride = I.block_table_seq_stride;
    p.scale_log2e = I.scale * 1.4426950408889634f;
    p.kernel_flags = I.kernel_flags;
    p.check_indices = (I.check_indices && I.kernel_flags != nullptr) ? 1 : 0;
    p.num_blocks = static_cast<long long>(I.num_blocks);
    return p;
}

bool checkIndicesFromEnv() {
    const char *v = std::getenv("INFINIOP_PAGED_CHECK_INDICES");
    return v != nullptr && v[0] == '1';
}

} // namespace b200::paged_attention

using b200::paged_attention::Descriptor;

__INFINI_C infiniStatus_t infiniopCreatePagedAttentionDescriptor(
    infiniopHandle_t handle,
    infiniopPagedAttentionDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    float scale) {
    B200_RETURN_IF(handle == nullptr || desc_ptr == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(out_desc == nullptr || q_desc == nullptr || k_cache_desc == nullptr || v_cache_desc == nullptr
                       || block_tables_desc == nullptr || seq_lens_desc == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(handle->device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);

    b200::paged_attention::Info info;
    infiniStatus_t st = b200::paged_attention::makeInfo(info, out_desc, q_desc, k_cache_desc, v_cache_desc,
                                                        block_tables_desc, seq_lens_desc, alibi_slopes_desc, scale);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    // Kernel-side index arithmetic uses int for counts.
    B200_RETURN_IF(info.num_seqs > 0x7fffffffu || info.num_heads > 65535u || info.max_num_blocks_per_seq > 0x7fffffffu
                       || info.block_size > 65536u || info.num_blocks > 0x7fffffffu,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);

    auto *h = reinterpret_cast<b200::Handle *>(handle);
    info.kernel_flags = h->props->kernel_flags;
    info.check_indices = b200::paged_attention::checkIndicesFromEnv();
    auto *d = new Descriptor{{handle->device, handle->device_id, b200::OpKind::PagedAttention, h->props}, info, {}, 0};

    // INFINIOP_PAGED_DECODE_PATH = auto (default) | stream | generic
    const char *path = std::getenv("INFINIOP_PAGED_DECODE_PATH");
    const bool force_generic = (path != nullptr) && std::strcmp(path, "generic") == 0;
    if (!force_generic) {
        d->stream = b200::paged_attention::planStream(info, *h->props);
    }
    if (path != nullptr && std::strcmp(path, "stream") == 0 && !d->stream.eligible) {
        std::fprintf(stderr, "[infiniop] INFINIOP_PAGED_DECODE_PATH=stream but this problem is not eligible for the streaming kernel\n");
        delete d;
        return INFINI_STATUS_BAD_PARAM;
    }
    d->workspace_bytes = d->stream.eligible ? d->stream.workspace_bytes : 0;
    *desc_ptr = reinterpret_cast<infiniopPagedAttentionDescriptor_t>(d);
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopGetPagedAttentionWorkspaceSize(
    infiniopPagedAttentionDescriptor_t desc, size_t *size) {
    B200_RETURN_IF(desc == nullptr || size == nullptr, INFINI_STATUS_NULL_POINTER);
    *size = reinterpret_cast<Descriptor *>(desc)->workspace_bytes;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopPagedAttention(
    infiniopPagedAttentionDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    const void *k_cache,
    const void *v_cache,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    void *stream) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<Descriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::PagedAttention, INFINI_STATUS_BAD_PARAM);
    const auto &I = d->info;
    if (I.num_seqs == 0 || I.num_heads == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    B200_RETURN_IF(out == nullptr || q == nullptr || k_cache == nullptr || v_cache == nullptr
                       || block_tables == nullptr || seq_lens == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(I.has_alibi && alibi_slopes == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(workspace_size < d->workspace_bytes, INFINI_STATUS_INSUFFICIENT_WORKSPACE);
    B200_RETURN_IF(d->workspace_bytes > 0 && workspace == nullptr, INFINI_STATUS_NULL_POINTER);

    const auto p = b200::paged_attention::makeDecodeParams(I, out, q, k_cache, v_cache, block_tables, seq_lens, alibi_slopes);
    auto cuda_stream = static_cast<cudaStream_t>(stream);
    if (d->stream.eligible) {
        return b200::paged_attention::launchDecodeStream(I, d->stream, p, workspace, workspace_size, cuda_stream);
    }
    return b200::paged_attention::launchDecodeGeneric(I, p, cuda_stream);
}

// No reference counterpart: the same call with every output row stored to several buffers of the
// descriptor's `out` shape and strides (outs[0] is the ordinary output).
__INFINI_C infiniStatus_t infiniopPagedAttentionMultiOut(
    infiniopPagedAttentionDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *const *outs,
    size_t num_outs,
    const void *q,
    const void *k_cache,
    const void *v_cache,
    const void *block_tables,
    const void *seq_lens,
    const void *alibi_slopes,
    void *stream) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<Descriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::PagedAttention, INFINI_STATUS_BAD_PARAM);
    B200_RETURN_IF(outs == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(num_outs < 1 || num_outs > 1 + b200::paged_attention::DecodeParams::kMaxExtraOut, INFINI_STATUS_BAD_PARAM);
    const auto &I = d->info;
    if (I.num_seqs == 0 || I.num_heads == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    for (size_t i = 0; i < num_outs; ++i) {
        B200_RETURN_IF(outs[i] == nullptr, INFINI_STATUS_NULL_POINTER);
    }
    B200_RETURN_IF(q == nullptr || k_cache == nullptr || v_cache == nullptr || block_tables == nullptr || seq_lens == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(I.has_alibi && alibi_slopes == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(workspace_size < d->workspace_bytes, INFINI_STATUS_INSUFFICIENT_WORKSPACE);
    B200_RETURN_IF(d->workspace_bytes > 0 && workspace == nullptr, INFINI_STATUS_NULL_POINTER);

    auto p = b200::paged_attention::makeDecodeParams(I, outs[0], q, k_cache, v_cache, block_tables, seq_lens, alibi_slopes);
    p.num_extra_out = static_cast<int>(num_outs) - 1;
    for (int i = 0; i < p.num_extra_out; ++i) {
        p.extra_out[i] = outs[i + 1];
    }
    auto cuda_stream = static_cast<cudaStream_t>(stream);
    if (d->stream.eligible) {
        return b200::paged_attention::launchDecodeStream(I, d->stream, p, workspace, workspace_size, cuda_stream);
    }
    return b200::paged_attention::launchDecodeGeneric(I, p, cuda_stream);
}

__INFINI_C infiniStatus_t infiniopDestroyPagedAttentionDescriptor(
    infiniopPagedAttentionDescriptor_t desc) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    delete reinterpret_cast<Descriptor *>(desc);
    return INFINI_STATUS_SUCCESS;
}
