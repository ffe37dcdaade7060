// Generic decode kernel: covers every shape the descriptor accepts (head sizes 64..576,
// value size != head size for the 576/512 latent-attention case, any block size, any cache
// strides, ALiBi).  It is the path for inputs the streaming kernel does not take; it is
// correct first and only moderately fast.  One CTA per (sequence, q-head); the row-wise
// attention itself lives in attend_row.cuh.
#include "attend_row.cuh"

namespace b200::paged_attention {

namespace {

template <typename T>
__global__ void __launch_bounds__(row::kWarps * 32)
    pagedDecodeGenericKernel(const DecodeParams p) {
    extern __shared__ float smem[];
    const int seq = blockIdx.x;
    const int head = blockIdx.y;
    const long long seq_len_ll = loadIndex(p.seq_lens, seq, p.index_is_64);
    if (seq_len_ll <= 0) {
        return; // output row stays untouched
    }
    const long long capacity = static_cast<long long>(p.max_blocks_per_seq) * p.block_size;
    const int seq_len = static_cast<int>(seq_len_ll > capacity ? capacity : seq_len_ll);
    const T *q = static_cast<const T *>(p.q) + seq * p.q_seq_stride + head * p.q_head_stride;
    T *out = static_cast<T *>(p.out) + seq * p.o_seq_stride + head * p.o_head_stride;
    row::attendRow<T>(p, q, out, head, head / p.group_size, seq * p.bt_seq_stride, seq_len, smem);
}

} // namespace

infiniStatus_t launchDecodeGeneric(const Info &info, const DecodeParams &p, cudaStream_t stream) {
    if (p.num_seqs == 0 || p.num_heads == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    // 2-element vector loads need even element strides on the caches.
    B200_RETURN_IF((p.k_block_stride | p.k_head_stride | p.k_row_stride | p.v_block_stride | p.v_head_stride | p.v_row_stride) & 1,
                   INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF((reinterpret_cast<uintptr_t>(p.k_cache) | reinterpret_cast<uintptr_t>(p.v_cache)) & 3, INFINI_STATUS_BAD_PARAM);
    B200_RETURN_IF(p.num_heads > 65535, INFINI_STATUS_BAD_TENSOR_SHAPE);
    const dim3 grid(p.num_seqs, p.num_heads);
    const dim3 block(row::kWarps * 32);
    const size_t smem = row::sharedBytes(p.head_size, p.value_size);
    // further destinations: the same launch again with its output redirected (this path is the
    // uncommon one; the streaming kernels store every destination themselves)
    for (int d = 0; d <= p.num_extra_out; ++d) {
        DecodeParams pd = p;
        pd.out = (d == 0) ? p.out : p.extra_out[d - 1];
        pd.num_extra_out = 0;
        if (info.dtype == INFINI_DTYPE_F16) {
            pagedDecodeGenericKernel<__half><<<grid, block, smem, stream>>>(pd);
        } else {
            pagedDecodeGenericKernel<__nv_bfloat16><<<grid, block, smem, stream>>>(pd);
        }
    }
    return checkLaunch("pagedDecodeGenericKernel");
}

} // namespace b200::paged_attention
