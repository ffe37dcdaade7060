// Row-wise attention shared by the generic decode kernel and the generic prefill kernel: one CTA
// (4 warps) computes one (query row, q-head) against the first `seq_len` tokens of a paged
// sequence.  Warp w walks tokens w, w+4, ...; lanes split the head dimension in pairs, a 5-step
// shuffle reduction produces the score, each warp keeps its own fp32 online-softmax state (m, l,
// acc) in the log2 domain, and the four states are merged through shared memory.
//
// The arithmetic is the one the reference kernels use
// (src/infiniop/ops/paged_attention/cuda/kernel_v2.cuh:134-336: scores * scale * log2e, exp2f, fp32
// accumulation), minus the +1e-6 in the final normalisation (l >= 1 always, so the term is below
// fp32 resolution of the result).  ALiBi: score += slope * (t - (seq_len - 1)).
#ifndef INFINIOP_B200_ATTEND_ROW_CUH
#define INFINIOP_B200_ATTEND_ROW_CUH

#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200::paged_attention::row {

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

inline size_t sharedBytes(int head_size, int value_size) {
    return sizeof(float) * (head_size + kWarps * (value_size + 2));
}

// smem layout: q[head_size] | per warp: m, l, acc[value_size].  Must be called by all kWarps * 32
// threads of the CTA with seq_len >= 1.
template <typename T>
__device__ inline void attendRow(const DecodeParams &p, const T *q, T *out, int head, int kv_head,
                                 long long bt_row, int seq_len, float *smem) {
    using T2 = typename Vec2<T>::type;
    float *q_s = smem;
    float *merge = smem + p.head_size;
    const int merge_stride = p.value_size + 2;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

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

    for (int t = warp; t < seq_len; t += kWarps) {
        const int logical_block = t / p.block_size;
        const int row = t - logical_block * p.block_size;
        const long long block = checkedBlock(p, loadIndex(p.block_tables, bt_row + logical_block, p.index_is_64));
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
    for (int d = threadIdx.x; d < p.value_size; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            o = fmaf(wgt[w], merge[w * merge_stride + 2 + d], o);
        }
        out[d] = fromFloat(o * inv_l, T());
    }
}

} // namespace b200::paged_attention::row

#endif
