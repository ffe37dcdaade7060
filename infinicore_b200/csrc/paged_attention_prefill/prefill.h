// Metadata and launch interface of infiniopPagedAttentionPrefill.
//
// Accepted inputs and status codes follow reference
// src/infiniop/ops/paged_attention_prefill/info.h:38-175.  The reference checks the three index
// tensors' dtypes one by one but instantiates its kernels on the block-table dtype for all of them
// (nvidia/paged_attention_prefill_nvidia.cu), so mixed index dtypes are refused here.
#ifndef INFINIOP_B200_PAGED_ATTENTION_PREFILL_H
#define INFINIOP_B200_PAGED_ATTENTION_PREFILL_H

#include "../paged_attention/kernels.h"

namespace b200::paged_attention_prefill {

struct Info {
    paged_attention::Info attn; // shapes/strides shared with decode; num_seqs = batch size here
    size_t total_q_tokens;
};

struct PrefillParams {
    paged_attention::DecodeParams d; // q/out strides are per TOKEN here; num_seqs = batch size
    const void *cum_seq_lens_q;
    int total_q;
};

inline infiniStatus_t makeInfo(Info &I,
                               infiniopTensorDescriptor_t out_desc,
                               infiniopTensorDescriptor_t q_desc,
                               infiniopTensorDescriptor_t k_cache_desc,
                               infiniopTensorDescriptor_t v_cache_desc,
                               infiniopTensorDescriptor_t block_tables_desc,
                               infiniopTensorDescriptor_t seq_lens_desc,
                               infiniopTensorDescriptor_t cum_seq_lens_q_desc,
                               infiniopTensorDescriptor_t alibi_slopes_desc,
                               float scale) {
    paged_attention::Info &A = I.attn;
    const infiniDtype_t dtype = q_desc->dtype;
    B200_RETURN_IF(dtype != INFINI_DTYPE_F16 && dtype != INFINI_DTYPE_BF16, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(out_desc->dtype != dtype || k_cache_desc->dtype != dtype || v_cache_desc->dtype != dtype,
                   INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(q_desc->ndim() != 3 || out_desc->ndim() != 3, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(k_cache_desc->ndim() != 4 || v_cache_desc->ndim() != 4, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(block_tables_desc->ndim() != 2 || seq_lens_desc->ndim() != 1 || cum_seq_lens_q_desc->ndim() != 1,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(q_desc->stride(2) != 1 || out_desc->stride(2) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF(k_cache_desc->stride(3) != 1 || v_cache_desc->stride(3) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);

    auto is_index = [](infiniDtype_t d) { return d == INFINI_DTYPE_I64 || d == INFINI_DTYPE_I32 || d == INFINI_DTYPE_U32; };
    const infiniDtype_t idx = block_tables_desc->dtype;
    B200_RETURN_IF(!is_index(idx) || !is_index(seq_lens_desc->dtype) || !is_index(cum_seq_lens_q_desc->dtype), INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(seq_lens_desc->dtype != idx || cum_seq_lens_q_desc->dtype != idx, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(block_tables_desc->stride(1) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF(seq_lens_desc->dim(0) > 1 && seq_lens_desc->stride(0) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF(cum_seq_lens_q_desc->stride(0) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);

    A.has_alibi = false;
    if (alibi_slopes_desc != nullptr) {
        B200_RETURN_IF(alibi_slopes_desc->dtype != INFINI_DTYPE_F32, INFINI_STATUS_BAD_TENSOR_DTYPE);
        B200_RETURN_IF(alibi_slopes_desc->ndim() != 1, INFINI_STATUS_BAD_TENSOR_SHAPE);
        B200_RETURN_IF(alibi_slopes_desc->stride(0) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
        A.has_alibi = true;
    }

    A.dtype = dtype;
    A.index_dtype = idx;
    A.scale = scale;
    I.total_q_tokens = q_desc->dim(0);
    A.num_heads = q_desc->dim(1);
    A.head_size = q_desc->dim(2);
    A.value_size = v_cache_desc->dim(3);
    A.num_blocks = k_cache_desc->dim(0);
    A.num_kv_heads = k_cache_desc->dim(1);
    A.block_size = k_cache_desc->dim(2);
    A.max_num_blocks_per_seq = block_tables_desc->dim(1);
    A.num_seqs = seq_lens_desc->dim(0);

    const bool is_mla = (A.head_size == 576 && A.value_size == 512);
    B200_RETURN_IF(A.head_size != 64 && A.head_size != 128 && A.head_size != 192 && A.head_size != 256 && A.head_size != 576,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(A.num_kv_heads == 0 || A.num_heads % A.num_kv_heads != 0, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(k_cache_desc->dim(3) != A.head_size, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(v_cache_desc->dim(0) != A.num_blocks || v_cache_desc->dim(1) != A.num_kv_heads || v_cache_desc->dim(2) != A.block_size,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(!is_mla && A.value_size != A.head_size, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(out_desc->dim(0) != q_desc->dim(0) || out_desc->dim(1) != q_desc->dim(1) || out_desc->dim(2) != A.value_size,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(cum_seq_lens_q_desc->dim(0) != A.num_seqs + 1, INFINI_STATUS_BAD_PARAM);
    B200_RETURN_IF(block_tables_desc->dim(0) != A.num_seqs, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(A.block_size == 0, INFINI_STATUS_BAD_TENSOR_SHAPE);

    A.q_seq_stride = q_desc->stride(0);
    A.q_head_stride = q_desc->stride(1);
    A.o_seq_stride = out_desc->stride(0);
    A.o_head_stride = out_desc->stride(1);
    A.k_block_stride = k_cache_desc->stride(0);
    A.k_head_stride = k_cache_desc->stride(1);
    A.k_row_stride = k_cache_desc->stride(2);
    A.v_block_stride = v_cache_desc->stride(0);
    A.v_head_stride = v_cache_desc->stride(1);
    A.v_row_stride = v_cache_desc->stride(2);
    A.block_table_seq_stride = block_tables_desc->stride(0);
    return INFINI_STATUS_SUCCESS;
}

// Row-wise path: every accepted shape.
infiniStatus_t launchPrefillGeneric(const Info &info, const PrefillParams &p, cudaStream_t stream);

// Tensor-core path (mma.sync, K/V staged by TMA); decided at descriptor creation.
struct TilePlan {
    bool eligible = false;
    int box_rows = 16; // rows of one TMA box: 16 when block_size % 16 == 0, else 8
    size_t smem_bytes = 0;
};
TilePlan planPrefillTiles(const Info &info, const DeviceProps &props);
infiniStatus_t launchPrefillTiles(const Info &info, const TilePlan &plan, const PrefillParams &p, cudaStream_t stream);

// Blackwell tensor-core path (tcgen05.mma, TMEM accumulators); head size 128.
struct UmmaPlan {
    bool eligible = false;
    int box_rows = 16;
    int stages = 2;  // slots of the V ring
    int k_stages = 3; // slots of the K ring (>= stages)
    int q_tiles = 1; // q-heads of one GQA group per CTA (share every staged KV tile)
    long long test_delay_v_cycles = 0; // test only: every V copy from the second tile on is held back this long
};
UmmaPlan planPrefillUmma(const Info &info, const DeviceProps &props);
infiniStatus_t launchPrefillUmma(const Info &info, const UmmaPlan &plan, const PrefillParams &p, cudaStream_t stream);

} // namespace b200::paged_attention_prefill

#endif
