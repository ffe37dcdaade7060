// Row-wise prefill kernel: one CTA per (query token, q-head).  A new token t of a chunk of n in a
// sequence of total length L is exactly a decode query against the first L - n + t + 1 tokens of
// that sequence, so the row-wise attention of the decode path (attend_row.cuh) is reused with a
// per-row length.  Covers every accepted shape; the tensor-core kernel takes the common ones.
#include "prefill.h"

#include "../paged_attention/attend_row.cuh"

namespace b200::paged_attention_prefill {

namespace {

namespace row = paged_attention::row;
using paged_attention::loadIndex;

template <typename T>
__global__ void __launch_bounds__(row::kWarps * 32)
    pagedPrefillGenericKernel(const PrefillParams pp) {
    extern __shared__ float smem[];
    const paged_attention::DecodeParams &p = pp.d;
    const long long token = blockIdx.x;
    const int head = blockIdx.y;

    // sequence that owns this packed token: last i with cum[i] <= token
    int lo = 0, hi = p.num_seqs;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (loadIndex(pp.cum_seq_lens_q, mid, p.index_is_64) <= token) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    const long long q_begin = loadIndex(pp.cum_seq_lens_q, lo, p.index_is_64);
    const long long q_end = loadIndex(pp.cum_seq_lens_q, lo + 1, p.index_is_64);
    if (token < q_begin || token >= q_end) {
        return; // token outside every chunk (cum does not cover it): leave the row untouched
    }
    const long long total = loadIndex(p.seq_lens, lo, p.index_is_64);
    long long allowed = total - (q_end - q_begin) + (token - q_begin) + 1;
    const long long capacity = static_cast<long long>(p.max_blocks_per_seq) * p.block_size;
    allowed = allowed > capacity ? capacity : allowed;
    if (allowed <= 0) {
        return;
    }
    const T *q = static_cast<const T *>(p.q) + token * p.q_seq_stride + head * p.q_head_stride;
    T *out = static_cast<T *>(p.out) + token * p.o_seq_stride + head * p.o_head_stride;
    row::attendRow<T>(p, q, out, head, head / p.group_size, lo * p.bt_seq_stride, static_cast<int>(allowed), smem);
}

} // namespace

infiniStatus_t launchPrefillGeneric(const Info &info, const PrefillParams &pp, cudaStream_t stream) {
    const auto &p = pp.d;
    if (pp.total_q == 0 || p.num_heads == 0 || p.num_seqs == 0) {
        return INFINI_STATUS_SUCCESS;
    }
    B200_RETURN_IF((p.k_block_stride | p.k_head_stride | p.k_row_stride | p.v_block_stride | p.v_head_stride | p.v_row_stride) & 1,
                   INFINI_STATUS_BAD_TENSOR_STRIDES);
    B200_RETURN_IF((reinterpret_cast<uintptr_t>(p.k_cache) | reinterpret_cast<uintptr_t>(p.v_cache)) & 3, INFINI_STATUS_BAD_PARAM);
    B200_RETURN_IF(p.num_heads > 65535, INFINI_STATUS_BAD_TENSOR_SHAPE);
    const dim3 grid(pp.total_q, p.num_heads);
    const dim3 block(row::kWarps * 32);
    const size_t smem = row::sharedBytes(p.head_size, p.value_size);
    if (info.attn.dtype == INFINI_DTYPE_F16) {
        pagedPrefillGenericKernel<__half><<<grid, block, smem, stream>>>(pp);
    } else {
        pagedPrefillGenericKernel<__nv_bfloat16><<<grid, block, smem, stream>>>(pp);
    }
    return checkLaunch("pagedPrefillGenericKernel");
}

} // namespace b200::paged_attention_prefill
