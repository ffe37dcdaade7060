// Generic decode kernel: covers every shape the descriptor accepts (head sizes 64..576,
// value size != head size for the 576/512 latent-attention case, any block size, any cache
// strides, ALiBi).  It is the path for inputs the streaming kernel does not take; it is
// correct first and only moderately fast.
//
// One CTA (4 warps) per (q-head, sequence).  Warp w walks tokens w, w+4, ...; lanes split
// the head dimension in pairs, a 5-step shuffle reduction produces the score, and each
// warp keeps its own fp32 online-softmax state (m, l, acc) in the log2 domain.  The four
// warp states are merged through shared memory at the end.  The arithmetic is the one the
// reference kernels use (src/infiniop/ops/paged_attention/cuda/kernel_v2.cuh:134-336:
// scores * scale * log2e, exp2f, fp32 accumulation), minus the +1e-6 in the final
// normalisation (l >= 1 always, so the term is below fp32 resolution of the result).
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200::paged_attention {

namespace {

constexpr int kWarps = 4;
constexpr int kMaxPairsPerLane = 9; // 576 / 64

__device__ inline float2 toFloat2(const __half2 v) { return __half22float2(v); }
__device__ inline float2 toFloat2(const __nv_bfloat162 v) { return __bfloat1622float2(v); }

template <typename T>
struct Vec2;
template <>
struct Vec2<__half> {
    using type = __half2;
};
template <>
struct Vec2<__nv_bfloat16> {
    using type = __nv_bfloat162;
};

__device__ inline __half fromFloat(float v, __half) { return __float2half_rn(v); }
__device__ inline __nv_bfloat16 fromFloat(float v, __nv_bfloat16) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
    pagedDecodeGenericKernel(const DecodeParams p) {
    using T2 = typename Vec2<T>::type;
    extern __shared__ float smem[];
    // layout: q[head_size] | per warp: m, l, acc[value_size]
    float *q_s = smem;
    float *merge = smem + p.head_size;
    const int merge_stride = p.value_size + 2;

    const int seq = blockIdx.x;
    const int head = blockIdx.y;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const long long seq_len_ll = loadIndex(p.seq_lens, seq, p.index_is_64);
    if (seq_len_ll <= 0) {
        return; // output row stays untouched
    }
    const int seq_len = static_cast<int>(seq_len_ll);
    const int kv_head = head / p.group_size;

    const T *q = static_cast<const T *>(p.q) + seq * p.q_seq_stride + head * p.q_head_stride;
    for (int i = threadIdx.x; i < p.head_size; i += blockDim.x) {
        q_s[i] = static_cast<float>(q[i]);
    }
    __syncthreads();

    const float slope_log2 = (p.alibi_slopes != nullptr) ? p.alibi_slopes[head] * 1.4426950408889634f : 0.f;

    float m = -INFINITY;
    float l = 0.f;
    float2 acc[kMaxPairsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPairsPerLane; ++i) {
        acc[i] = make_float2(0.f, 0.f);
    }

    const T *k_base = static_cast<const T *>(p.k_cache) + kv_head * p.k_head_stride;
    const T *v_base = static_cast<const T *>(p.v_cache) + kv_head * p.v_head_stride;
    const long long bt_row = seq * p.bt_seq_stride;

    for (int t = warp; t < seq_len; t += kWarps) {
        const int logical_block = t / p.block_size;
        const int row = t - logical_block * p.block_size;
        const long long block = loadIndex(p.block_tables, bt_row + logical_block, p.index_is_64);
        const T *k_row = k_base + block * p.k_block_stride + row * p.k_row_stride;
        const T *v_row = v_base + block * p.v_block_stride + row * p.v_row_stride;

        float dot = 0.f;
        for (int d = lane * 2; d < p.head_size; d += 64) {
            const float2 kk = toFloat2(*reinterpret_cast<const T2 *>(k_row + d));
            dot = fmaf(q_s[d], kk.x, dot);
            dot = fmaf(q_s[d + 1], kk.y, dot);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            dot += __shfl_xor_sync(0xffffffffu, dot, o);
        }
        float s = dot * p.scale_log2e;
        if (slope_log2 != 0.f) {
            s += slope_log2 * static_cast<float>(t - (seq_len - 1));
        }
        const float m_new = fmaxf(m, s);
        const float alpha = exp2f(m - m_new); // first token: exp2(-inf) = 0
        const float pr = exp2f(s - m_new);
        l = l * alpha + pr;
        m = m_new;
#pragma unroll
        for (int i = 0; i < kMaxPairsPerLane; ++i) {
            const int d = lane * 2 + i * 64;
            if (d < p.value_size) {
                const float2 vv = toFloat2(*reinterpret_cast<const T2 *>(v_row + d));
                acc[i].x = fmaf(pr, vv.x, acc[i].x * alpha);
                acc[i].y = fmaf(pr, vv.y, acc[i].y * alpha);
            }
        }
    }

    // merge the warp states
    float *mine = merge + warp * merge_stride;
    if (lane == 0) {
        mine[0] = m;
        mine[1] = l;
    }
#pragma unroll
    for (int i = 0; i < kMaxPairsPerLane; ++i) {
        const int d = lane * 2 + i * 64;
        if (d < p.value_size) {
            mine[2 + d] = acc[i].x;
            mine[2 + d + 1] = acc[i].y;
        }
    }
    __syncthreads();

    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        m_all = fmaxf(m_all, merge[w * merge_stride]);
    }
    float wgt[kWarps];
    float l_all = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const float mw = merge[w * merge_stride];
        wgt[w] = (mw == -INFINITY) ? 0.f : exp2f(mw - m_all);
        l_all += wgt[w] * merge[w * merge_stride + 1];
    }
    const float inv_l = 1.f / l_all;
    T *out = static_cast<T *>(p.out) + seq * p.o_seq_stride + head * p.o_head_stride;
    for (int d = threadIdx.x; d < p.value_size; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            o = fmaf(wgt[w], merge[w * merge_stride + 2 + d], o);
        }
        out[d] = fromFloat(o * inv_l, T());
    }
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
    const dim3 block(kWarps * 32);
    const size_t smem = sizeof(float) * (p.head_size + kWarps * (p.value_size + 2));
    if (info.dtype == INFINI_DTYPE_F16) {
        pagedDecodeGenericKernel<__half><<<grid, block, smem, stream>>>(p);
    } else {
        pagedDecodeGenericKernel<__nv_bfloat16><<<grid, block, smem, stream>>>(p);
    }
    return checkLaunch("pagedDecodeGenericKernel");
}

} // namespace b200::paged_attention
