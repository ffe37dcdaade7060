// Shape/stride metadata of one paged-attention problem, captured at descriptor creation.
//
// The accepted inputs and the status code returned for each rejected one follow
// reference src/infiniop/ops/paged_attention/info.h:41-194.  Two inputs the reference reads
// but never validates are honoured here instead of being assumed dense: the head stride of
// q (reference kernels index q as head * head_size, cuda/kernel_v2.cuh:180-181) and the row
// stride of block_tables (reference: seq * max_num_blocks_per_seq, cuda/kernel_v2.cuh:177).
#ifndef INFINIOP_B200_PAGED_ATTENTION_INFO_H
#define INFINIOP_B200_PAGED_ATTENTION_INFO_H

#include "../common.h"

namespace b200::paged_attention {

struct Info {
    infiniDtype_t dtype;       // F16 | BF16
    infiniDtype_t index_dtype; // I64 | I32 | U32 (block_tables and seq_lens agree)
    float scale;
    bool has_alibi;

    size_t num_seqs;
    size_t num_heads;
    size_t num_kv_heads;
    size_t head_size;
    size_t value_size;
    size_t block_size;
    size_t num_blocks;
    size_t max_num_blocks_per_seq;

    // element strides
    ptrdiff_t q_seq_stride, q_head_stride;
    ptrdiff_t o_seq_stride, o_head_stride;
    ptrdiff_t k_block_stride, k_head_stride, k_row_stride;
    ptrdiff_t v_block_stride, v_head_stride, v_row_stride;
    ptrdiff_t block_table_seq_stride;

    // set by the descriptor's creator, not by makeInfo: where the kernels report (the device's status word)
    // and whether they check block-table entries against the pool (INFINIOP_PAGED_CHECK_INDICES=1)
    unsigned int *kernel_flags = nullptr;
    bool check_indices = false;
};

inline infiniStatus_t makeInfo(Info &I,
                               infiniopTensorDescriptor_t out_desc,
                               infiniopTensorDescriptor_t q_desc,
                               infiniopTensorDescriptor_t k_cache_desc,
                               infiniopTensorDescriptor_t v_cache_desc,
                               infiniopTensorDescriptor_t block_tables_desc,
                               infiniopTensorDescriptor_t seq_lens_desc,
                               infiniopTensorDescriptor_t alibi_slopes_desc,
                               float scale) {
    const infiniDtype_t dtype = q_desc->dtype;
    B200_RETURN_IF(dtype != INFINI_DTYPE_F16 && dtype != INFINI_DTYPE_BF16, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(out_desc->dtype != dtype || k_cache_desc->dtype != dtype || v_cache_desc->dtype != dtype,
                   INFINI_STATUS_BAD_TENSOR_DTYPE);

    B200_RETURN_IF(q_desc->ndim() != 3 || out_desc->ndim() != 3, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(k_cache_desc->ndim() != 4 || v_cache_desc->ndim() != 4, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(block_tables_desc->ndim() != 2 || seq_lens_desc->ndim() != 1, INFINI_STATUS_BAD_TENSOR_SHAPE);

    B200_RETURN_IF(q_desc->stride(2) != 1 || out_desc->stride(2) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF(k_cache_desc->stride(3) != 1 || v_cache_desc->stride(3) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);

    const infiniDtype_t bt_dt = block_tables_desc->dtype;
    const infiniDtype_t sl_dt = seq_lens_desc->dtype;
    auto is_index = [](infiniDtype_t d) { return d == INFINI_DTYPE_I64 || d == INFINI_DTYPE_I32 || d == INFINI_DTYPE_U32; };
    B200_RETURN_IF(!is_index(bt_dt) || !is_index(sl_dt) || bt_dt != sl_dt, INFINI_STATUS_BAD_TENSOR_DTYPE);
    B200_RETURN_IF(block_tables_desc->stride(1) != 1 || seq_lens_desc->stride(0) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);

    I.has_alibi = false;
    if (alibi_slopes_desc != nullptr) {
        B200_RETURN_IF(alibi_slopes_desc->dtype != INFINI_DTYPE_F32, INFINI_STATUS_BAD_TENSOR_DTYPE);
        B200_RETURN_IF(alibi_slopes_desc->ndim() != 1, INFINI_STATUS_BAD_TENSOR_SHAPE);
        B200_RETURN_IF(alibi_slopes_desc->stride(0) != 1, INFINI_STATUS_BAD_TENSOR_STRIDES);
        I.has_alibi = true;
    }

    I.dtype = dtype;
    I.index_dtype = bt_dt;
    I.scale = scale;
    I.num_seqs = q_desc->dim(0);
    I.num_heads = q_desc->dim(1);
    I.head_size = q_desc->dim(2);
    I.value_size = v_cache_desc->dim(3);
    I.num_blocks = k_cache_desc->dim(0);
    I.num_kv_heads = k_cache_desc->dim(1);
    I.block_size = k_cache_desc->dim(2);
    I.max_num_blocks_per_seq = block_tables_desc->dim(1);

    const bool is_mla = (I.head_size == 576 && I.value_size == 512);
    B200_RETURN_IF(I.head_size != 64 && I.head_size != 128 && I.head_size != 192 && I.head_size != 256 && I.head_size != 576,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(I.num_kv_heads == 0 || I.num_heads % I.num_kv_heads != 0, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(k_cache_desc->dim(3) != I.head_size, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(v_cache_desc->dim(0) != k_cache_desc->dim(0) || v_cache_desc->dim(1) != k_cache_desc->dim(1) || v_cache_desc->dim(2) != k_cache_desc->dim(2),
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(!is_mla && I.value_size != I.head_size, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(out_desc->dim(0) != I.num_seqs || out_desc->dim(1) != I.num_heads || out_desc->dim(2) != I.value_size,
                   INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(seq_lens_desc->dim(0) != I.num_seqs, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(block_tables_desc->dim(0) != I.num_seqs, INFINI_STATUS_BAD_TENSOR_SHAPE);
    B200_RETURN_IF(I.block_size == 0, INFINI_STATUS_BAD_TENSOR_SHAPE);
    if (I.has_alibi) {
        B200_RETURN_IF(alibi_slopes_desc->dim(0) != I.num_heads, INFINI_STATUS_BAD_TENSOR_SHAPE);
    }

    I.q_seq_stride = q_desc->stride(0);
    I.q_head_stride = q_desc->stride(1);
    I.o_seq_stride = out_desc->stride(0);
    I.o_head_stride = out_desc->stride(1);
    I.k_block_stride = k_cache_desc->stride(0);
    I.k_head_stride = k_cache_desc->stride(1);
    I.k_row_stride = k_cache_desc->stride(2);
    I.v_block_stride = v_cache_desc->stride(0);
    I.v_head_stride = v_cache_desc->stride(1);
    I.v_row_stride = v_cache_desc->stride(2);
    I.block_table_seq_stride = block_tables_desc->stride(0);
    return INFINI_STATUS_SUCCESS;
}

} // namespace b200::paged_attention

#endif
