// C entry points of infiniopPagedAttentionPrefill.  Replaces reference
// src/infiniop/ops/paged_attention_prefill/operator.cc and
// nvidia/paged_attention_prefill_nvidia.cu (descriptor, workspace, dispatch).  Workspace size is 0:
// neither kernel of this library splits a query tile's KV range across CTAs.
#include "prefill.h"

#include <cstdlib>
#include <cstring>

namespace b200::paged_attention_prefill {

struct Descriptor {
    OpDescriptorBase base;
    Info info;
    TilePlan tiles;
    UmmaPlan umma;
};

} // namespace b200::paged_attention_prefill

using b200::paged_attention_prefill::Descriptor;

__INFINI_C infiniStatus_t infiniopCreatePagedAttentionPrefillDescriptor(
    infiniopHandle_t handle,
    infiniopPagedAttentionPrefillDescriptor_t *desc_ptr,
    infiniopTensorDescriptor_t out_desc,
    infiniopTensorDescriptor_t q_desc,
    infiniopTensorDescriptor_t k_cache_desc,
    infiniopTensorDescriptor_t v_cache_desc,
    infiniopTensorDescriptor_t block_tables_desc,
    infiniopTensorDescriptor_t seq_lens_desc,
    infiniopTensorDescriptor_t cum_seq_lens_q_desc,
    infiniopTensorDescriptor_t alibi_slopes_desc,
    float scale) {
    B200_RETURN_IF(handle == nullptr || desc_ptr == nullptr, INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(out_desc == nullptr || q_desc == nullptr || k_cache_desc == nullptr || v_cache_desc == nullptr
                       || block_tables_desc == nullptr || seq_lens_desc == nullptr || cum_seq_lens_q_desc == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(handle->device != INFINI_DEVICE_NVIDIA, INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED);

    b200::paged_attention_prefill::Info info;
    infiniStatus_t st = b200::paged_attention_prefill::makeInfo(info, out_desc, q_desc, k_cache_desc, v_cache_desc, block_tables_desc,
                                                                seq_lens_desc, cum_seq_lens_q_desc, alibi_slopes_desc, scale);
    B200_RETURN_IF(st != INFINI_STATUS_SUCCESS, st);
    const auto &A = info.attn;
    B200_RETURN_IF(A.num_seqs > 0x7fffffffu || info.total_q_tokens > 0x7fffffffu || A.num_heads > 65535u
                       || A.max_num_blocks_per_seq > 0x7fffffffu || A.block_size > 65536u || A.num_blocks > 0x7fffffffu,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);

    auto *h = reinterpret_cast<b200::Handle *>(handle);
    info.attn.kernel_flags = h->props->kernel_flags;
    info.attn.check_indices = b200::paged_attention::checkIndicesFromEnv();
    auto *d = new Descriptor{{handle->device, handle->device_id, b200::OpKind::PagedAttentionPrefill, h->props}, info, {}, {}};
    // INFINIOP_PAGED_PREFILL_PATH = auto (default) | umma | tiles | generic
    const char *path = std::getenv("INFINIOP_PAGED_PREFILL_PATH");
    const bool want_generic = path != nullptr && std::strcmp(path, "generic") == 0;
    const bool want_tiles = path != nullptr && std::strcmp(path, "tiles") == 0;
    const bool want_umma = path != nullptr && std::strcmp(path, "umma") == 0;
    if (!want_generic) {
        d->tiles = b200::paged_attention_prefill::planPrefillTiles(info, *h->props);
    }
    if (want_umma || path == nullptr || std::strcmp(path, "auto") == 0) {
        d->umma = b200::paged_attention_prefill::planPrefillUmma(info, *h->props);
        if (want_umma && !d->umma.eligible) {
            std::fprintf(stderr, "[infiniop] INFINIOP_PAGED_PREFILL_PATH=umma but this problem is not eligible for the tcgen05 kernel\n");
            delete d;
            return INFINI_STATUS_BAD_PARAM;
        }
    }
    (void)want_tiles;
    if (path != nullptr && std::strcmp(path, "tiles") == 0 && !d->tiles.eligible) {
        std::fprintf(stderr, "[infiniop] INFINIOP_PAGED_PREFILL_PATH=tiles but this problem is not eligible for the tensor-core kernel\n");
        delete d;
        return INFINI_STATUS_BAD_PARAM;
    }
    *desc_ptr = reinterpret_cast<infiniopPagedAttentionPrefillDescriptor_t>(d);
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopGetPagedAttentionPrefillWorkspaceSize(
    infiniopPagedAttentionPrefillDescriptor_t desc, size_t *size) {
    B200_RETURN_IF(desc == nullptr || size == nullptr, INFINI_STATUS_NULL_POINTER);
    *size = 0;
    return INFINI_STATUS_SUCCESS;
}

__INFINI_C infiniStatus_t infiniopPagedAttentionPrefill(
    infiniopPagedAttentionPrefillDescriptor_t desc,
    void *workspace,
    size_t workspace_size,
    void *out,
    const void *q,
    const void *k_cache,
    const void *v_cache,
    const void *block_tables,
    const void *seq_lens,
    const void *cum_seq_lens_q,
    const void *alibi_slopes,
    void *stream) {
    (void)workspace;
    (void)workspace_size;
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    auto *d = reinterpret_cast<Descriptor *>(desc);
    B200_RETURN_IF(d->base.kind != b200::OpKind::PagedAttentionPrefill, INFINI_STATUS_BAD_PARAM);
    const auto &A = d->info.attn;
    if (d->info.total_q_tokens == 0 || A.num_heads == 0 || A.num_seqs == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    B200_RETURN_IF(out == nullptr || q == nullptr || k_cache == nullptr || v_cache == nullptr || block_tables == nullptr
                       || seq_lens == nullptr || cum_seq_lens_q == nullptr,
                   INFINI_STATUS_NULL_POINTER);
    B200_RETURN_IF(A.has_alibi && alibi_slopes == nullptr, INFINI_STATUS_NULL_POINTER);

    b200::paged_attention_prefill::PrefillParams pp;
    auto &p = pp.d;
    p.out = out;
    p.q = q;
    p.k_cache = k_cache;
    p.v_cache = v_cache;
    p.block_tables = block_tables;
    p.seq_lens = seq_lens;
    p.alibi_slopes = A.has_alibi ? static_cast<const float *>(alibi_slopes) : nullptr;
    p.num_seqs = static_cast<int>(A.num_seqs);
    p.num_heads = static_cast<int>(A.num_heads);
    p.num_kv_heads = static_cast<int>(A.num_kv_heads);
    p.group_size = static_cast<int>(A.num_heads / A.num_kv_heads);
    p.head_size = static_cast<int>(A.head_size);
    p.value_size = static_cast<int>(A.value_size);
    p.block_size = static_cast<int>(A.block_size);
    p.max_blocks_per_seq = static_cast<int>(A.max_num_blocks_per_seq);
    p.index_is_64 = (A.index_dtype == INFINI_DTYPE_I64) ? 1 : 0;
    p.q_seq_stride = A.q_seq_stride;
    p.q_head_stride = A.q_head_stride;
    p.o_seq_stride = A.o_seq_stride;
    p.o_head_stride = A.o_head_stride;
    p.k_block_stride = A.k_block_stride;
    p.k_head_stride = A.k_head_stride;
    p.k_row_stride = A.k_row_stride;
    p.v_block_stride = A.v_block_stride;
    p.v_head_stride = A.v_head_stride;
    p.v_row_stride = A.v_row_stride;
    p.bt_seq_stride = A.block_table_seq_stride;
    p.scale_log2e = A.scale * 1.4426950408889634f;
    p.kernel_flags = A.kernel_flags;
    p.check_indices = (A.check_indices && A.kernel_flags != nullptr) ? 1 : 0;
    p.num_blocks = static_cast<long long>(A.num_blocks);
    pp.cum_seq_lens_q = cum_seq_lens_q;
    pp.total_q = static_cast<int>(d->info.total_q_tokens);

    auto cuda_stream = static_cast<cudaStream_t>(stream);
    if (d->umma.eligible) {
        return b200::paged_attention_prefill::launchPrefillUmma(d->info, d->umma, pp, cuda_stream);
    }
    if (d->tiles.eligible) {
        return b200::paged_attention_prefill::launchPrefillTiles(d->info, d->tiles, pp, cuda_stream);
    }
    return b200::paged_attention_prefill::launchPrefillGeneric(d->info, pp, cuda_stream);
}

__INFINI_C infiniStatus_t infiniopDestroyPagedAttentionPrefillDescriptor(
    infiniopPagedAttentionPrefillDescriptor_t desc) {
    B200_RETURN_IF(desc == nullptr, INFINI_STATUS_NULL_POINTER);
    delete reinterpret_cast<Descriptor *>(desc);
    return INFINI_STATUS_SUCCESS;
}
