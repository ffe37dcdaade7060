// Tensor-core prefill kernel for sm_100a: FlashAttention-style forward over a paged KV cache.
//
// What it computes is what the reference's prefill kernels compute
// (src/infiniop/ops/paged_attention_prefill/cuda/kernel_v2.cuh): for new token t of a chunk of n in
// a sequence of total KV length L, softmax over KV positions 0 .. L - n + t of scale * q.k, times V,
// fp32 online softmax in the log2 domain.
//
// Shape of the kernel:
//  * one CTA = one (sequence, q-head, tile of 64 new tokens).  The host does not know the chunk
//    lengths, so the grid is sized to an upper bound (ceil(total_q / 64) + num_seqs tiles) and each
//    CTA finds its (sequence, first token) with a block scan over cum_seq_lens_q.
//  * 4 consumer warps own 16 query rows each; a 5th warp is the producer.  The producer walks the
//    sequence's KV in tiles of 64 tokens, looks up the block table (one entry per lane) and issues
//    non-multicast `cp.async.bulk.tensor` boxes (64 elements x 8 or 16 rows, 128-byte swizzle) into
//    a ring of shared-memory stages; a "full" mbarrier per stage tracks the bytes, an "empty"
//    mbarrier per stage hands the stage back.
//  * consumers run S = Q.K^T and O += P.V as mma.sync.m16n8k16 (bf16/fp16 in, fp32 accumulate) with
//    ldmatrix / ldmatrix.trans operand loads, P rounded to the cache dtype as the reference's torch
//    check does.  A warp skips KV tiles that lie entirely above its rows' causal limit.
//  * every wait is an mbarrier wait on this CTA's own copies or on its own warps, bounded by a
//    timeout; no CTA waits on another.
#include "prefill.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

namespace b200::paged_attention_prefill {

namespace {

using paged_attention::DecodeParams;
using paged_attention::loadIndex;

constexpr int kBM = 64;              // query rows per CTA
constexpr int kBN = 64;              // KV tokens per stage
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kStages = 2;
constexpr long long kWaitLimitCycles = 4000000000ll; // an mbarrier wait gives up after ~2 s

__device__ __forceinline__ uint32_t smemAddr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarInit(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: false means the limit ran out (the copy or MMA it waits for never completed).  The
// bound is counted on the SM's cycle counter, which is cheap to read; roughly 2 s at 2 GHz.
__device__ __forceinline__ bool mbarWait(uint32_t bar, uint32_t parity) {
    if (mbarTryWait(bar, parity)) {
        return true;
    }
    const long long t0 = clock64();
    while (!mbarTryWait(bar, parity)) {
        if (clock64() - t0 > kWaitLimitCycles) {
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tmaLoadBox(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void ldmatrixX4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrixX4Trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fastExp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t packPair(float lo, float hi, __nv_bfloat16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t packPair(float lo, float hi, __half) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
// named barrier among the consumer warps only
__device__ __forceinline__ void consumerSync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}

struct TileArgs {
    PrefillParams pp;
    int box_rows; // 8 or 16
    unsigned int *error; // the device's status word (infiniopGetKernelStatus); may be null
};

template <typename T, int HD>
__global__ void __launch_bounds__(kThreads)
    pagedPrefillTileKernel(const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v,
                           const TileArgs a) {
    constexpr int kChunks = HD / 64;
    constexpr int kTensorBytes = kChunks * kBN * 128; // one K (or V) tile: [chunk][64 rows][128 B], swizzled
    constexpr int kStageBytes = 2 * kTensorBytes;
    constexpr int kKSteps = HD / 16;
    constexpr int kNTiles = HD / 8;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // all shared memory is carved from the dynamic block so the swizzled tiles keep their 1024-byte
    // alignment: [stages x (K tile | V tile)] [full barriers] [empty barriers] [scan scratch]
    int *scratch = reinterpret_cast<int *>(smem_raw + kStages * kStageBytes + 2 * kStages * 8);
    int &sh_seq = scratch[0];
    int &sh_t0 = scratch[1];
    int &sh_found = scratch[2];
    int *sh_warp_tot = scratch + 4;

    const DecodeParams &p = a.pp.d;
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int head = blockIdx.y;
    const int tile_id = blockIdx.x;

    const uint32_t ring = smemAddr(smem_raw);
    const uint32_t full_bar = ring + kStages * kStageBytes;
    const uint32_t empty_bar = full_bar + kStages * 8;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbarInit(full_bar + s * 8, 1);
            mbarInit(empty_bar + s * 8, kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        sh_found = 0;
    }
    __syncthreads();

    // ---- which (sequence, first new token) is this tile? ----------------------------------------
    {
        int carry = 0;
        for (int base = 0; base < p.num_seqs; base += kThreads) {
            const int i = base + tid;
            int tiles = 0;
            if (i < p.num_seqs) {
                const long long n = loadIndex(a.pp.cum_seq_lens_q, i + 1, p.index_is_64) - loadIndex(a.pp.cum_seq_lens_q, i, p.index_is_64);
                tiles = n > 0 ? static_cast<int>((n + kBM - 1) / kBM) : 0;
            }
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) {
                    incl += v;
                }
            }
            if (lane == 31) {
                sh_warp_tot[warp] = incl;
            }
            __syncthreads();
            int prev = 0, total = 0;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) {
                prev += (w < warp) ? sh_warp_tot[w] : 0;
                total += sh_warp_tot[w];
            }
            const int excl = carry + prev + incl - tiles;
            if (tiles > 0 && tile_id >= excl && tile_id < excl + tiles) {
                sh_seq = i;
                sh_t0 = (tile_id - excl) * kBM;
                sh_found = 1;
            }
            __syncthreads();
            if (sh_found) {
                break;
            }
            carry += total;
        }
    }
    if (!sh_found) {
        return;
    }
    const int seq = sh_seq;
    const int t0 = sh_t0;
    const long long q_begin = loadIndex(a.pp.cum_seq_lens_q, seq, p.index_is_64);
    const int n_new = static_cast<int>(loadIndex(a.pp.cum_seq_lens_q, seq + 1, p.index_is_64) - q_begin);
    const long long capacity = static_cast<long long>(p.max_blocks_per_seq) * p.block_size;
    long long total_ll = loadIndex(p.seq_lens, seq, p.index_is_64);
    total_ll = total_ll > capacity ? capacity : total_ll;
    const int total_len = static_cast<int>(total_ll);
    const int cache_len = total_len - n_new;
    const int rows_valid = min(kBM, n_new - t0);
    // KV positions this tile can see: [0, kv_end)
    const int kv_end = min(total_len, cache_len + t0 + rows_valid);
    if (kv_end <= 0) {
        return;
    }
    const int num_kv_tiles = (kv_end + kBN - 1) / kBN;
    const int kv_head = head / p.group_size;

    if (warp == kConsumerWarps) {
        // ================================ producer warp ==========================================
        const int box_rows = a.box_rows;
        const int boxes_per_tensor = (kBN / box_rows) * kChunks;
        const int box_bytes = box_rows * 128;
        for (int kt = 0; kt < num_kv_tiles; ++kt) {
            const int stage = kt % kStages;
            const uint32_t parity = (kt / kStages) & 1;
            if (kt >= kStages) {
                if (!mbarWait(empty_bar + stage * 8, parity ^ 1u)) {
                    if (lane == 0 && a.error != nullptr) {
                        atomicOr(a.error, 1u);
                    }
                    return;
                }
            }
            const int kv0 = kt * kBN;
            // sub-tiles of box_rows tokens whose first token exists get copied; the rest of the stage
            // keeps stale bytes that the consumers mask (K) or zero (V)
            const int live_sub = min(kBN / box_rows, (kv_end - kv0 + box_rows - 1) / box_rows);
            const uint32_t dst = ring + stage * kStageBytes;
            if (lane == 0) {
                mbarExpectTx(full_bar + stage * 8, static_cast<uint32_t>(2 * live_sub * kChunks * box_bytes));
            }
            __syncwarp();
            for (int b = lane; b < 2 * boxes_per_tensor; b += 32) {
                const int is_v = b / boxes_per_tensor;
                const int r = (b % boxes_per_tensor) / kChunks; // sub-tile
                const int c = b % kChunks;
                if (r < live_sub) {
                    const int j0 = kv0 + r * box_rows;
                    const int page = j0 / p.block_size;
                    const int row0 = j0 - page * p.block_size;
                    const long long block = paged_attention::reportedBlock(p, loadIndex(p.block_tables, seq * p.bt_seq_stride + page, p.index_is_64));
                    tmaLoadBox(dst + is_v * kTensorBytes + c * (kBN * 128) + r * box_bytes, is_v ? &tmap_v : &tmap_k,
                               full_bar + stage * 8, c * 64, row0, kv_head, static_cast<int>(block));
                }
            }
        }
        return;
    }

    // ==================================== consumer warps =========================================
    const int g = lane >> 2;
    const int t = lane & 3;
    const int row_a = warp * 16 + g;      // tile-local query rows of this thread
    const int row_b = row_a + 8;
    const int limit_a = cache_len + t0 + row_a; // last KV position row a may see
    const int limit_b = limit_a + 8;
    const int warp_limit_max = cache_len + t0 + warp * 16 + 15;

    uint32_t qa[kKSteps][4];
    {
        const long long tok_a = q_begin + t0 + row_a;
        const long long tok_b = tok_a + 8;
        const bool va = row_a < rows_valid, vb = row_b < rows_valid;
        const T *qa_ptr = static_cast<const T *>(p.q) + tok_a * p.q_seq_stride + head * p.q_head_stride;
        const T *qb_ptr = static_cast<const T *>(p.q) + tok_b * p.q_seq_stride + head * p.q_head_stride;
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
            qa[ks][0] = va ? *reinterpret_cast<const uint32_t *>(qa_ptr + ks * 16 + 2 * t) : 0u;
            qa[ks][1] = vb ? *reinterpret_cast<const uint32_t *>(qb_ptr + ks * 16 + 2 * t) : 0u;
            qa[ks][2] = va ? *reinterpret_cast<const uint32_t *>(qa_ptr + ks * 16 + 8 + 2 * t) : 0u;
            qa[ks][3] = vb ? *reinterpret_cast<const uint32_t *>(qb_ptr + ks * 16 + 8 + 2 * t) : 0u;
        }
    }
    const float slope_log2 = (p.alibi_slopes != nullptr) ? p.alibi_slopes[head] * 1.4426950408889634f : 0.f;

    float o[kNTiles][4];
#pragma unroll
    for (int n = 0; n < kNTiles; ++n) {
        o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    bool failed = false;

    for (int kt = 0; kt < num_kv_tiles; ++kt) {
        const int stage = kt % kStages;
        const uint32_t parity = (kt / kStages) & 1;
        const uint32_t k_tile = ring + stage * kStageBytes;
        const uint32_t v_tile = k_tile + kTensorBytes;
        const int kv0 = kt * kBN;
        if (!mbarWait(full_bar + stage * 8, parity)) {
            failed = true;
            break;
        }
        const int valid = kv_end - kv0; // KV tokens of this stage that exist for this tile
        if (valid < kBN) {
            // V rows past the end may hold anything: zero them (0 * NaN would poison the accumulators)
            for (int idx = tid; idx < (kBN - valid) * kChunks * 8; idx += kConsumerWarps * 32) {
                const int row = valid + idx / (kChunks * 8);
                const int rest = idx % (kChunks * 8);
                const uint32_t addr = v_tile + (rest / 8) * (kBN * 128) + row * 128 + (rest % 8) * 16;
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            consumerSync();
        }

        if (kv0 <= warp_limit_max) { // otherwise every position of the stage is above this warp's causal limit
            // ---- S = Q . K^T : 16 rows x 64 KV tokens ---------------------------------------------
            float s[kBN / 8][4];
#pragma unroll
            for (int n = 0; n < kBN / 8; ++n) {
                s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
            }
            {
                const int l_row = ((lane >> 4) << 3) + (lane & 7);
                const int l_half = (lane >> 3) & 1;
#pragma unroll
                for (int ks = 0; ks < kKSteps; ++ks) {
                    const int col = ks * 2 + l_half;
#pragma unroll
                    for (int nb = 0; nb < kBN / 16; ++nb) {
                        const int row = nb * 16 + l_row;
                        const uint32_t addr = k_tile + (col >> 3) * (kBN * 128) + row * 128 + (((col & 7) ^ (row & 7)) << 4);
                        uint32_t b0, b1, b2, b3;
                        ldmatrixX4(addr, b0, b1, b2, b3);
                        mma16816<T>(s[2 * nb], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                        mma16816<T>(s[2 * nb + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
                    }
                }
            }

            // ---- online softmax (log2 domain) for rows a and b -------------------------------------
            const bool need_mask = (kv0 + kBN - 1 > limit_a) || (valid < kBN);
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int n = 0; n < kBN / 8; ++n) {
                const int j = kv0 + n * 8 + 2 * t;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float xa = s[n][e] * p.scale_log2e;
                    float xb = s[n][2 + e] * p.scale_log2e;
                    if (slope_log2 != 0.f) {
                        xa += slope_log2 * static_cast<float>(j + e - limit_a);
                        xb += slope_log2 * static_cast<float>(j + e - limit_b);
                    }
                    if (need_mask) {
                        xa = (j + e <= limit_a && j + e < kv_end) ? xa : -INFINITY;
                        xb = (j + e <= limit_b && j + e < kv_end) ? xb : -INFINITY;
                    }
                    s[n][e] = xa;
                    s[n][2 + e] = xb;
                    mx_a = fmaxf(mx_a, xa);
                    mx_b = fmaxf(mx_b, xb);
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a);
            const float mn_b = fmaxf(m_b, mx_b);
            // a row whose every position so far is masked keeps m = -inf; use 0 as the subtrahend there
            const float sub_a = (mn_a == -INFINITY) ? 0.f : mn_a;
            const float sub_b = (mn_b == -INFINITY) ? 0.f : mn_b;
            const float alpha_a = fastExp2(m_a - sub_a);
            const float alpha_b = fastExp2(m_b - sub_b);
            m_a = mn_a;
            m_b = mn_b;
            uint32_t pa[kBN / 16][4];
            float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
            for (int n = 0; n < kBN / 8; ++n) {
                const float p0 = fastExp2(s[n][0] - sub_a);
                const float p1 = fastExp2(s[n][1] - sub_a);
                const float p2 = fastExp2(s[n][2] - sub_b);
                const float p3 = fastExp2(s[n][3] - sub_b);
                sum_a += p0 + p1;
                sum_b += p2 + p3;
                pa[n >> 1][(n & 1) * 2] = packPair(p0, p1, T());
                pa[n >> 1][(n & 1) * 2 + 1] = packPair(p2, p3, T());
            }
            l_a = l_a * alpha_a + sum_a;
            l_b = l_b * alpha_b + sum_b;
#pragma unroll
            for (int n = 0; n < kNTiles; ++n) {
                o[n][0] *= alpha_a;
                o[n][1] *= alpha_a;
                o[n][2] *= alpha_b;
                o[n][3] *= alpha_b;
            }

            // ---- O += P . V ------------------------------------------------------------------------
            {
                const int l_row = (((lane >> 3) & 1) << 3) + (lane & 7);
                const int l_sel = lane >> 4;
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk) {
#pragma unroll
                    for (int np = 0; np < kNTiles / 2; ++np) {
                        const int col = np * 2 + l_sel;
                        const int row = kk * 16 + l_row;
                        const uint32_t addr = v_tile + (col >> 3) * (kBN * 128) + row * 128 + (((col & 7) ^ (row & 7)) << 4);
                        uint32_t b0, b1, b2, b3;
                        ldmatrixX4Trans(addr, b0, b1, b2, b3);
                        mma16816<T>(o[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                        mma16816<T>(o[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                    }
                }
            }
        }

        // hand the stage back to the producer
        __syncwarp();
        if (lane == 0) {
            mbarArrive(empty_bar + stage * 8);
        }
    }

    if (failed) {
        if (lane == 0 && a.error != nullptr) {
            atomicOr(a.error, 1u);
        }
        return;
    }

    // ---- normalise and store ---------------------------------------------------------------------
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    if (row_a < rows_valid) {
        const float inv = l_a > 0.f ? 1.f / l_a : 0.f;
        T *out = static_cast<T *>(p.out) + (q_begin + t0 + row_a) * p.o_seq_stride + head * p.o_head_stride;
#pragma unroll
        for (int n = 0; n < kNTiles; ++n) {
            *reinterpret_cast<uint32_t *>(out + n * 8 + 2 * t) = packPair(o[n][0] * inv, o[n][1] * inv, T());
        }
    }
    if (row_b < rows_valid) {
        const float inv = l_b > 0.f ? 1.f / l_b : 0.f;
        T *out = static_cast<T *>(p.out) + (q_begin + t0 + row_b) * p.o_seq_stride + head * p.o_head_stride;
#pragma unroll
        for (int n = 0; n < kNTiles; ++n) {
            *reinterpret_cast<uint32_t *>(out + n * 8 + 2 * t) = packPair(o[n][2] * inv, o[n][3] * inv, T());
        }
    }
}

// ---- host -------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encodeTiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess
            && qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        } else {
            (void)cudaGetLastError();
        }
    });
    return fn;
}

bool encodeCacheMap(CUtensorMap *map, const paged_attention::Info &A, const void *base, ptrdiff_t row_stride,
                    ptrdiff_t head_stride, ptrdiff_t block_stride, size_t width, int box_rows) {
    EncodeTiledFn fn = encodeTiled();
    if (fn == nullptr) {
        return false;
    }
    const cuuint64_t dims[4] = {width, A.block_size, A.num_kv_heads, A.num_blocks};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(row_stride) * 2, static_cast<cuuint64_t>(head_stride) * 2,
                                   static_cast<cuuint64_t>(block_stride) * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = (A.dtype == INFINI_DTYPE_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    return fn(map, dt, 4, const_cast<void *>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int HD>
infiniStatus_t launchTyped(const TilePlan &plan, const TileArgs &args, const CUtensorMap &mk, const CUtensorMap &mv,
                           unsigned tiles, int device_id, cudaStream_t stream) {
    static std::mutex attr_mutex;
    static size_t attr_bytes[64] = {};
    auto kernel = pagedPrefillTileKernel<T, HD>;
    {
        std::lock_guard<std::mutex> lock(attr_mutex);
        const bool tracked = device_id >= 0 && device_id < 64;
        if (!tracked || attr_bytes[device_id] < plan.smem_bytes) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes)) != cudaSuccess) {
                return checkLaunch("cudaFuncSetAttribute(pagedPrefillTileKernel)");
            }
            if (tracked) {
                attr_bytes[device_id] = plan.smem_bytes;
            }
        }
    }
    const dim3 grid(tiles, args.pp.d.num_heads);
    kernel<<<grid, kThreads, plan.smem_bytes, stream>>>(mk, mv, args);
    return checkLaunch("pagedPrefillTileKernel");
}

} // namespace

TilePlan planPrefillTiles(const Info &info, const DeviceProps &props) {
    TilePlan plan;
    const auto &A = info.attn;
    const size_t hd = A.head_size;
    if (A.value_size != hd || (hd != 64 && hd != 128)) {
        return plan;
    }
    if (A.block_size % 8 != 0 || A.num_seqs == 0 || A.num_seqs > 65536 || info.total_q_tokens == 0 || A.num_blocks == 0) {
        return plan;
    }
    plan.box_rows = (A.block_size % 16 == 0) ? 16 : 8;
    auto even = [](ptrdiff_t v) { return (v & 1) == 0; };
    auto mult8 = [](ptrdiff_t v) { return v > 0 && (v % 8) == 0; };
    if (!even(A.q_seq_stride) || !even(A.q_head_stride) || !even(A.o_seq_stride) || !even(A.o_head_stride)) {
        return plan;
    }
    if (!mult8(A.k_row_stride) || !mult8(A.k_head_stride) || !mult8(A.k_block_stride)
        || !mult8(A.v_row_stride) || !mult8(A.v_head_stride) || !mult8(A.v_block_stride)) {
        return plan;
    }
    CUtensorMap probe;
    void *fake = reinterpret_cast<void *>(static_cast<uintptr_t>(1) << 30);
    if (!encodeCacheMap(&probe, A, fake, A.k_row_stride, A.k_head_stride, A.k_block_stride, hd, plan.box_rows)
        || !encodeCacheMap(&probe, A, fake, A.v_row_stride, A.v_head_stride, A.v_block_stride, hd, plan.box_rows)) {
        return plan;
    }
    plan.smem_bytes = static_cast<size_t>(kStages) * 2 * (hd / 64) * kBN * 128 + 2 * kStages * 8 + 1024;
    if (plan.smem_bytes > props.smem_per_block_optin) {
        return plan;
    }
    plan.eligible = true;
    return plan;
}

infiniStatus_t launchPrefillTiles(const Info &info, const TilePlan &plan, const PrefillParams &pp, cudaStream_t stream) {
    const auto &A = info.attn;
    const auto &p = pp.d;
    const auto addr = [](const void *ptr) { return reinterpret_cast<uintptr_t>(ptr); };
    if (((addr(p.k_cache) | addr(p.v_cache)) & 15u) != 0 || ((addr(p.q) | addr(p.out)) & 3u) != 0) {
        return launchPrefillGeneric(info, pp, stream);
    }
    CUtensorMap mk, mv;
    B200_RETURN_IF(!encodeCacheMap(&mk, A, p.k_cache, A.k_row_stride, A.k_head_stride, A.k_block_stride, A.head_size, plan.box_rows), INFINI_STATUS_INTERNAL_ERROR);
    B200_RETURN_IF(!encodeCacheMap(&mv, A, p.v_cache, A.v_row_stride, A.v_head_stride, A.v_block_stride, A.value_size, plan.box_rows), INFINI_STATUS_INTERNAL_ERROR);
    TileArgs args;
    args.pp = pp;
    args.box_rows = plan.box_rows;
    args.error = pp.d.kernel_flags;
    const unsigned tiles = static_cast<unsigned>((info.total_q_tokens + kBM - 1) / kBM + A.num_seqs);
    int device_id = -1;
    (void)cudaGetDevice(&device_id);
    const bool f16 = (A.dtype == INFINI_DTYPE_F16);
    if (A.head_size == 64) {
        return f16 ? launchTyped<__half, 64>(plan, args, mk, mv, tiles, device_id, stream)
                   : launchTyped<__nv_bfloat16, 64>(plan, args, mk, mv, tiles, device_id, stream);
    }
    return f16 ? launchTyped<__half, 128>(plan, args, mk, mv, tiles, device_id, stream)
               : launchTyped<__nv_bfloat16, 128>(plan, args, mk, mv, tiles, device_id, stream);
}

} // namespace b200::paged_attention_prefill
