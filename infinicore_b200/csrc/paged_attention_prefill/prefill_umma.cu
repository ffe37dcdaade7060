// Blackwell tensor-core prefill kernel: tcgen05.mma with TMEM accumulators, operands staged by TMA.
//
// Same result as prefill_tiles.cu (and the reference's prefill kernels,
// src/infiniop/ops/paged_attention_prefill/cuda/kernel_v2.cuh), different machine mapping:
//
//  * one CTA = one (sequence, q-head, tile of 128 new tokens).  Q tile [128 x 128] and the KV tiles
//    [64 tokens x 128] land in shared memory through non-multicast `cp.async.bulk.tensor` boxes with
//    the 128-byte swizzle, which is exactly the canonical K-major (Q, K) / MN-major (V) operand layout
//    of `tcgen05.mma`, so the MMA reads them through shared-memory descriptors with no repacking.
//  * S[128 x 64] = Q.K^T is 8 `tcgen05.mma.cta_group::1.kind::f16` (M=128, N=64, K=16) issued by one
//    thread of the score-issuing warp into one of two 64-column S buffers in TMEM; completion reaches
//    the other warps through `tcgen05.commit` on an mbarrier.
//  * thread r of the four softmax warps owns query row r: it reads its S row with `tcgen05.ld`
//    (32x32b: TMEM lane = row), does the fp32 online softmax without any cross-thread traffic, rounds
//    P to the cache dtype and stores it back over the scores it came from (`tcgen05.st`, two 16-bit
//    values per column): P never touches shared memory.
//  * O[128 x 128] += P.V is 4 more `tcgen05.mma` (M=128, N=128, K=16; A operand P read from TMEM, B
//    operand V from shared memory) issued by a second warp, accumulating in TMEM columns [128, 256)
//    across all KV tiles.  The running maximum used for the exponentials is only raised when a row's
//    true maximum exceeds it by more than 2^8 (the result is unchanged: numerator and denominator share
//    the same reference); only then does a warp read its O rows back, scale them and store them
//    (`tcgen05.ld` / `tcgen05.st`).  O is read once more at the end for the normalised store.  The
//    commits of the two issuing warps also release the K and V ring slots to the producers, and P.V of
//    tile i overlaps the S MMA and softmax arithmetic of tile i + 1.
//  * two more warps are the TMA producers (block-table lookups, K/V boxes; K copies run one tile ahead
//    of the V copies).  The first MMA warp owns the TMEM allocation.
//
// Every wait is an mbarrier wait with a time limit; on every path the CTA reaches the common exit,
// where the TMEM columns are released.
#include "prefill.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

namespace b200::paged_attention_prefill {

namespace {

using paged_attention::DecodeParams;
using paged_attention::loadIndex;

constexpr int kBM = 128;                 // query rows per CTA = MMA M
constexpr int kBN = 64;                  // KV tokens per stage = MMA N of S, K extent of P.V
// per head size HD (64 or 128): HD / 64 column chunks of 128 bytes per row; a Q tile is
// (HD / 64) * 128 rows * 128 B (32 KiB at head 128), a K or V tile (HD / 64) * 64 rows * 128 B (16 KiB)
constexpr int qTileBytes(int hd) { return (hd / 64) * kBM * 128; }
constexpr int kvTileBytes(int hd) { return (hd / 64) * kBN * 128; }
constexpr long long kWaitLimitCycles = 4000000000ll; // an mbarrier wait gives up after ~2 s

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smemAddr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
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
__device__ __forceinline__ void tmaLoad4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tmaLoad3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Shared memory -> global through a tensor map (clipped at the tensor's bounds); completion is tracked
// by the issuing thread's bulk-async group.
__device__ __forceinline__ void tmaStore3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tmaStoreCommitAndWaitRead() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void prefetchTensorMap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tcgenFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgenFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgenCommit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool electOne() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues it
__device__ __forceinline__ void ummaF16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]: A is read from tensor memory (row = lane, two 16-bit
// elements of the K extent per 32-bit column); one thread issues it
__device__ __forceinline__ void ummaF16FromTmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane, raw bits
__device__ __forceinline__ void tmemStoreBits32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmemLoad32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = __uint_as_float(r[i]);
    }
}
__device__ __forceinline__ void tmemStore32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 64 consecutive fp32 columns of this thread's TMEM lane: both loads in flight, then one wait.  The
// wait names the registers so that nothing reads them before it.
__device__ __forceinline__ void tmemLoad64(uint32_t taddr, float (&v)[64]) {
    uint32_t r[64];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t *q = r + 32 * h;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]),
              "=r"(q[8]), "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15]),
              "=r"(q[16]), "=r"(q[17]), "=r"(q[18]), "=r"(q[19]), "=r"(q[20]), "=r"(q[21]), "=r"(q[22]), "=r"(q[23]),
              "=r"(q[24]), "=r"(q[25]), "=r"(q[26]), "=r"(q[27]), "=r"(q[28]), "=r"(q[29]), "=r"(q[30]), "=r"(q[31])
            : "r"(taddr + 32 * h)
            : "memory");
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t *q = r + 32 * h;
        asm volatile(
            "tcgen05.wait::ld.sync.aligned;"
            : "+r"(q[0]), "+r"(q[1]), "+r"(q[2]), "+r"(q[3]), "+r"(q[4]), "+r"(q[5]), "+r"(q[6]), "+r"(q[7]),
              "+r"(q[8]), "+r"(q[9]), "+r"(q[10]), "+r"(q[11]), "+r"(q[12]), "+r"(q[13]), "+r"(q[14]), "+r"(q[15]),
              "+r"(q[16]), "+r"(q[17]), "+r"(q[18]), "+r"(q[19]), "+r"(q[20]), "+r"(q[21]), "+r"(q[22]), "+r"(q[23]),
              "+r"(q[24]), "+r"(q[25]), "+r"(q[26]), "+r"(q[27]), "+r"(q[28]), "+r"(q[29]), "+r"(q[30]), "+r"(q[31])
            :
            : "memory");
    }
#pragma unroll
    for (int i = 0; i < 64; ++i) {
        v[i] = __uint_as_float(r[i]);
    }
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Maximum of 64 values in 32 three-input instructions, 5 levels deep.
__device__ __forceinline__ float rowMax64(const float (&s)[64]) {
    float a[22], b[8];
#pragma unroll
    for (int j = 0; j < 21; ++j) {
        a[j] = max3(s[3 * j], s[3 * j + 1], s[3 * j + 2]);
    }
    a[21] = s[63];
#pragma unroll
    for (int j = 0; j < 7; ++j) {
        b[j] = max3(a[3 * j], a[3 * j + 1], a[3 * j + 2]);
    }
    b[7] = a[21];
    return max3(max3(b[0], b[1], b[2]), max3(b[3], b[4], b[5]), fmaxf(b[6], b[7]));
}
// Two fp32 lanes per instruction (packed f32x2 arithmetic of sm_100): halves the FMA-pipe
// instruction count of the per-element work.
__device__ __forceinline__ void fma2(float &d0, float &d1, float a0, float a1, float b, float c) {
    asm("{\n"
        ".reg .b64 ra, rb, rc, rd;\n"
        "mov.b64 ra, {%2, %3};\n"
        "mov.b64 rb, {%4, %4};\n"
        "mov.b64 rc, {%5, %5};\n"
        "fma.rn.f32x2 rd, ra, rb, rc;\n"
        "mov.b64 {%0, %1}, rd;\n"
        "}\n"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float &d0, float &d1, float a0, float a1) {
    asm("{\n"
        ".reg .b64 ra, rd;\n"
        "mov.b64 ra, {%2, %3};\n"
        "mov.b64 rd, {%0, %1};\n"
        "add.rn.f32x2 rd, rd, ra;\n"
        "mov.b64 {%0, %1}, rd;\n"
        "}\n"
        : "+f"(d0), "+f"(d1)
        : "f"(a0), "f"(a1));
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
// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
// Offsets are in bytes; the hardware fields drop the 4 low bits.
__device__ __forceinline__ uint64_t smemDesc(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor of kind::f16: fp32 accumulate, A/B both `fmt` (0 = f16, 1 = bf16).
__host__ __device__ constexpr uint32_t instrDesc(uint32_t fmt, uint32_t a_mn_major, uint32_t b_mn_major, uint32_t m, uint32_t n) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

struct UmmaArgs {
    PrefillParams pp;
    int box_rows;  // rows of one K/V TMA box: the largest of 64, 32, 16, 8 that divides block_size
    int tma_store; // out's strides allow a tensor map: full tiles leave through shared memory and one bulk store
    long long test_delay_v_cycles; // test only (0 in normal use): the V copies are held back this many cycles
};

// smem layout (dynamic, 1024-aligned):
//   [Q: kQ x 32 KiB][K ring: stages x 16 KiB][V ring: stages x 16 KiB][barriers][tmem base][scratch]
// TMEM columns of q-tile i (base + i * 256): S buffer 0 [0,64)  S buffer 1 [64,128)  O [128,256); the
// probabilities of a tile overwrite the first 32 columns of the S buffer their scores came from (two
// 16-bit values per column) and feed P.V from there as its A operand - P never touches shared memory.
//
// kQ q-heads of one GQA group (same 128 token rows) share every staged KV tile: with kQ = 2 each
// byte brought in from L2 feeds twice the math and eight softmax warps keep the special-function
// units busy while the tensor core works.  kQ = 1 is the same kernel for odd group sizes.
//
// Warp roles: softmax warps [0, 4 kQ) (warp w serves q-tile w / 4; thread owns query row
// (w % 4) * 32 + lane = its TMEM lane), then 2 kQ MMA-issuing warps (per q-tile one for the scores and
// one for P.V; the first also owns the TMEM allocation) and 2 kQ TMA producer warps (each stages its share of every K/V tile's pages, so
// neither the copies' issue cost nor the tensor-core instructions' issue cost sits in one warp).
// They talk through mbarriers only:
//   k_full/v_full[stage]   producers -> MMA (bytes landed; one arrival per producer warp)
//   k_empty/v_empty[stage] MMA -> producers (tcgen05.commit, one per MMA warp)
//   s_ready[i][buf]        score MMA i -> softmax i (S retired)     s_free[i][buf]  P.V MMA i -> score MMA i (P consumed)
//   p_ready[i][buf]        softmax i -> MMA i (P stored, 4 arrivals) o_done[i]      MMA i -> softmax i (P.V retired)
// (p_ready is one barrier per S buffer like the other two: the softmax may be two tiles ahead of P.V - P of
// tiles kt + 1 and kt + 2 stored while P.V of tile kt + 1 still waits for its V tile - and a waiter that is two
// phases behind a single barrier reads its parity wrongly and waits for ever; per buffer the softmax cannot
// store P of tile kt + 2 before P.V of tile kt has retired.)
// The score warp runs ahead of the softmax as far as the two S buffers allow, so the tensor core works
// on the next scores while the softmax warps are busy with the current ones.
template <typename T, int kStages, int kKStages, int kQ, int kHD>
__global__ void __launch_bounds__((8 * kQ) * 32)
    pagedPrefillUmmaKernel(const __grid_constant__ CUtensorMap tmap_q,
                           const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v,
                           const __grid_constant__ CUtensorMap tmap_o,
                           const UmmaArgs a) {
    constexpr int kSoftmaxWarpsAll = 4 * kQ;
    constexpr int kMmaWarp0 = kSoftmaxWarpsAll;      // MMA warps [4 kQ, 6 kQ): S issuers, then P.V issuers
    constexpr int kProducers = 2 * kQ;
    constexpr int kProducerWarp0 = 6 * kQ;           // producer warps [6 kQ, 8 kQ)
    constexpr int kNT = 8 * kQ * 32;
    constexpr int kTmemCols = 256 * kQ;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int kChunks = kHD / 64;
    constexpr int kQBytes = qTileBytes(kHD);
    constexpr int kTensorBytes = kvTileBytes(kHD);
    constexpr int kRingOff = kQ * kQBytes;
    constexpr int kBarOff = kRingOff + (kKStages + kStages) * kTensorBytes; // K ring [kKStages], then V ring [kStages]
    const uint32_t smem0 = smemAddr(smem_raw);
    const uint32_t q_tiles = smem0;
    const uint32_t ring = smem0 + kRingOff;
    const uint32_t k_full = smem0 + kBarOff;              // [kKStages]
    const uint32_t k_empty = k_full + kKStages * 8;       // [kKStages]
    const uint32_t v_full = k_empty + kKStages * 8;       // [kStages]
    const uint32_t v_empty = v_full + kStages * 8;        // [kStages]
    const uint32_t s_ready = v_empty + kStages * 8;       // [kQ][2]
    const uint32_t s_free = s_ready + kQ * 16;            // [kQ][2]
    const uint32_t p_ready = s_free + kQ * 16;            // [kQ][2]
    const uint32_t o_done = p_ready + kQ * 16;            // [kQ]
    const uint32_t drain_bar = o_done + kQ * 8;           // [2 kQ]
    const uint32_t q_bar = drain_bar + 2 * kQ * 8;
    constexpr int kNumBars = 2 * kKStages + 2 * kStages + 9 * kQ + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_raw + kBarOff + kNumBars * 8);
    int *scratch = reinterpret_cast<int *>(tmem_slot + 2);
    int &sh_seq = scratch[0];
    int &sh_t0 = scratch[1];
    int &sh_found = scratch[2];
    int &sh_failed = scratch[3];
    int &sh_n_new = scratch[4];
    int &sh_total_len = scratch[5];
    long long &sh_q_begin = *reinterpret_cast<long long *>(scratch + 6); // 8-byte aligned: the barriers and the TMEM slot before it are
    int *sh_warp_tot = scratch + 8;

    const DecodeParams &p = a.pp.d;
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int head0 = blockIdx.y * kQ; // first q-head of this CTA; all kQ heads read the same kv-head
    const int tile_id = blockIdx.x;

    if (tid == 0) {
        prefetchTensorMap(&tmap_q);
        prefetchTensorMap(&tmap_k);
        prefetchTensorMap(&tmap_v);
        for (int s = 0; s < kKStages; ++s) {
            mbarInit(k_full + s * 8, kProducers);
            mbarInit(k_empty + s * 8, kQ);
        }
        for (int s = 0; s < kStages; ++s) {
            mbarInit(v_full + s * 8, kProducers);
            mbarInit(v_empty + s * 8, kQ);
        }
        for (int i = 0; i < kQ; ++i) {
            for (int b = 0; b < 2; ++b) {
                mbarInit(s_ready + (i * 2 + b) * 8, 1);
                mbarInit(s_free + (i * 2 + b) * 8, 1);
            }
            mbarInit(p_ready + (i * 2) * 8, 4);
            mbarInit(p_ready + (i * 2 + 1) * 8, 4);
            mbarInit(o_done + i * 8, 1);
            mbarInit(drain_bar + i * 8, 1);
            mbarInit(drain_bar + (kQ + i) * 8, 1);
        }
        mbarInit(q_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        sh_found = 0;
        sh_failed = 0;
    }
    // TMEM: the first MMA warp allocates while the others look for the CTA's tile; everyone reads the base address
    // after the barriers of the search.  (A CTA past the last tile gives its columns back at the common exit.)
    if (warp == kMmaWarp0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tcgenFenceBefore();
    }
    __syncthreads();

    // ---- which (sequence, first new token) is this tile? ---------------------------------------------
    {
        int carry = 0;
        for (int base = 0; base < p.num_seqs; base += kNT) {
            const int i = base + tid;
            int tiles = 0;
            long long my_begin = 0, my_n = 0, my_len = 0;
            if (i < p.num_seqs) {
                // all three loads in flight together; the sequence that owns this tile publishes them below
                my_begin = loadIndex(a.pp.cum_seq_lens_q, i, p.index_is_64);
                my_n = loadIndex(a.pp.cum_seq_lens_q, i + 1, p.index_is_64) - my_begin;
                my_len = loadIndex(p.seq_lens, i, p.index_is_64);
                tiles = my_n > 0 ? static_cast<int>((my_n + kBM - 1) / kBM) : 0;
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
            for (int w = 0; w < kNT / 32; ++w) {
                prev += (w < warp) ? sh_warp_tot[w] : 0;
                total += sh_warp_tot[w];
            }
            const int excl = carry + prev + incl - tiles;
            if (tiles > 0 && tile_id >= excl && tile_id < excl + tiles) {
                const long long capacity = static_cast<long long>(p.max_blocks_per_seq) * p.block_size;
                sh_seq = i;
                sh_t0 = (tile_id - excl) * kBM;
                sh_q_begin = my_begin;
                sh_n_new = static_cast<int>(my_n);
                sh_total_len = static_cast<int>(my_len > capacity ? capacity : my_len);
                sh_found = 1;
            }
            __syncthreads();
            if (sh_found) {
                break;
            }
            carry += total;
        }
    }
    const bool found = sh_found != 0;
    const int seq = sh_seq;
    const int t0 = sh_t0;
    const long long q_begin = sh_q_begin;
    const int n_new = sh_n_new;
    const int total_len = sh_total_len;
    const int cache_len = total_len - n_new;
    const int rows_valid = min(kBM, n_new - t0);
    const int kv_end = min(total_len, cache_len + t0 + rows_valid);
    const bool skip = !found || kv_end <= 0; // nothing to do: straight to the common exit, where TMEM is released
    const int num_kv_tiles = (kv_end + kBN - 1) / kBN;
    const int kv_head = head0 / p.group_size;
    tcgenFenceAfter();
    const uint32_t tmem_base = *tmem_slot;

    if (skip) {
    } else if (warp >= kProducerWarp0) {
        // ================================ TMA producers ==========================================
        // A K/V tile is kBN / box_rows boxes of rows (one page or part of one) times kChunks column
        // chunks, per tensor.  Producer r takes row groups r, r + kProducers, ...; inside the warp one
        // lane owns one (row group, chunk) box, looks its page up in the block table one tile ahead
        // and issues the K copy and the V copy of that box.
        const int r = warp - kProducerWarp0;
        if (r == 0 && lane == 0) {
            mbarExpectTx(q_bar, kQ * kQBytes);
            for (int i = 0; i < kQ; ++i) {
                for (int c = 0; c < kChunks; ++c) {
                    tmaLoad3d(q_tiles + i * kQBytes + c * (kBM * 128), &tmap_q, q_bar, c * 64, head0 + i, static_cast<int>(q_begin + t0));
                }
            }
        }
        const int box_rows = a.box_rows;
        const int groups = kBN / box_rows;                   // row groups per tile
        const uint32_t box_bytes = static_cast<uint32_t>(box_rows) * 128u;
        const int my_group = r + (lane / kChunks) * kProducers;
        const int my_chunk = lane % kChunks;
        const bool has_box = my_group < groups;
        const long long bt_row = seq * p.bt_seq_stride;
        // (block, first row inside it) of this lane's box in tile kt; block < 0: nothing to copy
        auto locateBox = [&](int kt, long long &block, int &row0) {
            const int j0 = kt * kBN + my_group * box_rows;
            block = -1;
            row0 = 0;
            if (has_box && kt < num_kv_tiles && j0 < kv_end) {
                const int page = j0 / p.block_size;
                row0 = j0 - page * p.block_size;
                block = paged_attention::reportedBlock(p, loadIndex(p.block_tables, bt_row + page, p.index_is_64));
            }
        };
        // One tile's K (is_v = 0) or V copies of this warp: wait for the slot, announce the bytes, issue.
        auto issueTile = [&](int is_v, int kt, long long block, int row0) -> bool {
            const int depth = is_v ? kStages : kKStages;
            const int stage = kt % depth;
            const uint32_t parity = (kt / depth) & 1;
            const uint32_t full = (is_v ? v_full : k_full) + stage * 8;
            const uint32_t empty = (is_v ? v_empty : k_empty) + stage * 8;
            const bool live = block >= 0;
            const uint32_t bytes = static_cast<uint32_t>(__popc(__ballot_sync(0xffffffffu, live))) * box_bytes;
            if (is_v && kt >= 1 && a.test_delay_v_cycles > 0) {
                // test only: a V tile that arrives late lets the softmax run two tiles ahead of the P.V issuer -
                // the situation in which a single P-ready barrier for both score buffers is read wrongly
                const long long t_begin = clock64();
                while (clock64() - t_begin < a.test_delay_v_cycles) {
                }
            }
            if (kt >= depth && !__all_sync(0xffffffffu, mbarWait(empty, parity ^ 1u))) {
                return false;
            }
            if (lane == 0) {
                mbarExpectTx(full, bytes); // this warp's arrival, announcing its share of the tile
            }
            __syncwarp();
            if (live) {
                const uint32_t dst = ring + (is_v * kKStages + stage) * kTensorBytes + my_chunk * (kBN * 128) + my_group * box_bytes;
                tmaLoad4d(dst, is_v ? &tmap_v : &tmap_k, full, my_chunk * 64, row0, kv_head, static_cast<int>(block));
            }
            return true;
        };
        // The K copies run one tile ahead of the V copies: the scores of tile kt + 1 are wanted while the
        // softmax still works on tile kt, its values a whole tile later, and a V slot only frees when P.V two
        // tiles back has retired - K(kt + 1) must not queue behind that wait.  (A K slot frees when the scores
        // kKStages tiles back have retired, which is long before.)  Page-table entries are fetched two tiles
        // ahead of their first use.
        long long block0, block1, block2;
        int row00, row01, row02;
        locateBox(0, block0, row00);
        locateBox(1, block1, row01);
        int issued_k = 0, issued_v = 0;
        bool ok = issueTile(0, 0, block0, row00);
        if (ok) {
            issued_k = 1;
        }
        for (int kt = 0; kt < num_kv_tiles && ok; ++kt) {
            locateBox(kt + 2, block2, row02); // in flight while this step's copies are issued
            if (kt + 1 < num_kv_tiles) {
                ok = issueTile(0, kt + 1, block1, row01);
                if (!ok) {
                    break;
                }
                issued_k = kt + 2;
            }
            ok = issueTile(1, kt, block0, row00);
            if (!ok) {
                break;
            }
            issued_v = kt + 1;
            block0 = block1;
            row00 = row01;
            block1 = block2;
            row01 = row02;
        }
        if (!ok) {
            sh_failed = 1;
            // bounded wait for the copies of the last tiles this warp issued (as many as each ring holds)
            for (int kt = max(0, issued_k - kKStages); kt < issued_k; ++kt) {
                (void)mbarWait(k_full + (kt % kKStages) * 8, (kt / kKStages) & 1);
            }
            for (int kt = max(0, issued_v - kStages); kt < issued_v; ++kt) {
                (void)mbarWait(v_full + (kt % kStages) * 8, (kt / kStages) & 1);
            }
        }
    } else if (warp >= kMmaWarp0) {
        // ================================ MMA issuers ==============================================
        // Two warps per q-tile: one issues the score MMAs (S = Q.K^T, up to two tiles ahead of the
        // softmax - as far as the two S buffers allow), the other the P.V MMAs.  Separate warps keep a
        // wait for the softmax out of the way of the next scores.  In each, the whole warp walks the loop
        // in step and waits on the barriers; one elected lane issues the tensor-core instructions.
        {
            const int w = warp - kMmaWarp0;
            const int i = w % kQ;
            const bool scores = w < kQ;
            constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u; // 0 = f16, 1 = bf16
            constexpr uint32_t kIdescS = instrDesc(kFmt, 0, 0, kBM, kBN);  // Q (K-major) x K (K-major)
            constexpr uint32_t kIdescO = instrDesc(kFmt, 0, 1, kBM, kHD);  // P (K-major) x V (MN-major)
            // descriptors differ only in their start-address field: build one per operand and add
            const uint64_t q_desc = smemDesc(q_tiles + i * kQBytes, 16, 1024);
            const uint64_t k_desc = smemDesc(ring, 16, 1024);
            const uint64_t v_desc = smemDesc(ring + kKStages * kTensorBytes, kBN * 128, 1024);
            const uint32_t tmem_q = __shfl_sync(0xffffffffu, tmem_base, 0) + i * 256;
            const uint32_t my_s_ready = s_ready + i * 16;
            auto waitAll = [&](uint32_t bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbarWait(bar, parity)); };
            bool ok = true;
            if (scores) {
                ok = waitAll(q_bar, 0);
                for (int kt = 0; kt < num_kv_tiles && ok; ++kt) {
                    const int stage = kt % kKStages;
                    // The S buffer also holds P of tile kt - 2 (written over the scores it came from): P.V of
                    // that tile must have retired before new scores land there.  (A barrier per buffer: its
                    // next arrival needs these very scores, so it is never more than one phase ahead.)
                    ok = waitAll(k_full + stage * 8, (kt / kKStages) & 1)
                         && (kt < 2 || waitAll(s_free + (i * 2 + (kt & 1)) * 8, ((kt >> 1) - 1) & 1));
                    if (!ok) {
                        break;
                    }
                    tcgenFenceAfter();
                    const uint64_t kd = k_desc + ((stage * kTensorBytes) >> 4);
                    const uint32_t d = tmem_q + (kt & 1) * kBN;
                    if (electOne()) {
#pragma unroll
                        for (int ks = 0; ks < kHD / 16; ++ks) {
                            // 16 elements = 32 bytes inside the 128-byte swizzled row; 4 k-steps per 64-wide chunk
                            const uint32_t qo = ((ks / 4) * (kBM * 128) + (ks % 4) * 32) >> 4;
                            const uint32_t ko = ((ks / 4) * (kBN * 128) + (ks % 4) * 32) >> 4;
                            ummaF16(d, q_desc + qo, kd + ko, kIdescS, ks > 0 ? 1u : 0u);
                        }
                        tcgenCommit(my_s_ready + (kt & 1) * 8);
                        tcgenCommit(k_empty + stage * 8); // the K slot is free once every q-tile's S has retired
                    }
                    __syncwarp();
                }
            } else {
                for (int kt = 0; kt < num_kv_tiles && ok; ++kt) {
                    const int stage = kt % kStages;
                    ok = waitAll(v_full + stage * 8, (kt / kStages) & 1) && waitAll(p_ready + (i * 2 + (kt & 1)) * 8, (kt >> 1) & 1);
                    if (!ok) {
                        break;
                    }
                    tcgenFenceAfter();
                    const uint64_t vd = v_desc + ((stage * kTensorBytes) >> 4);
                    if (electOne()) {
#pragma unroll
                        for (int kk = 0; kk < kBN / 16; ++kk) {
                            // P: 16 of the K extent = 8 columns of the score buffer it was written over
                            ummaF16FromTmem(tmem_q + 128, tmem_q + (kt & 1) * kBN + kk * 8, vd + ((kk * 16 * 128) >> 4), kIdescO,
                                            (kt > 0 || kk > 0) ? 1u : 0u);
                        }
                        tcgenCommit(o_done + i * 8);
                        tcgenCommit(s_free + (i * 2 + (kt & 1)) * 8); // this tile's S / P buffer may take new scores
                        tcgenCommit(v_empty + stage * 8); // the V slot is free once every q-tile's P.V has retired
                    }
                    __syncwarp();
                }
            }
            if (!ok) {
                sh_failed = 1;
            }
            // whatever this warp issued must retire before TMEM and shared memory are given back
            if (electOne()) {
                tcgenCommit(drain_bar + w * 8);
            }
            __syncwarp();
            (void)waitAll(drain_bar + w * 8, 0);
        }
    } else {
        // ================================ softmax warps ==========================================
        const int qi = warp >> 2;                                      // q-tile (= q-head of the pair) this warp serves
        const int row = (warp & 3) * 32 + lane;                        // tile-local query row = TMEM lane
        const int head = head0 + qi;
        const int limit = cache_len + t0 + row;                        // last KV position this row may see
        const float slope_log2 = (p.alibi_slopes != nullptr) ? p.alibi_slopes[head] * 1.4426950408889634f : 0.f;
        const uint32_t lane_field = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tmem_q = tmem_base + qi * 256;
        const uint32_t tmem_o = tmem_q + 128;
        const uint32_t my_s_ready = s_ready + qi * 16;
        const uint32_t my_p_ready = p_ready + qi * 16, my_o_done = o_done + qi * 8;
        const int gtid = tid & 127;                                    // thread index within this q-tile's four warps
        const float c_log2 = p.scale_log2e;

        // Running reference maximum used for the exponentials (log2 domain) and the row sum.  The
        // reference is raised lazily, so p can reach 2^kLazyBits: far inside fp32 / bf16 / fp16 range
        // for the products that follow (fp16 P is bounded by 2^8).
        constexpr float kLazyBits = 8.f;
        float m_used = 0.f, l_run = 0.f;
        bool ok = true;

        for (int kt = 0; kt < num_kv_tiles; ++kt) {
            const int stage = kt % kStages;
            const int kv0 = kt * kBN;
            const int valid = kv_end - kv0;
            const uint32_t tmem_s = tmem_q + (kt & 1) * kBN;
            const uint32_t v_tile = ring + (kKStages + stage) * kTensorBytes;

            ok = mbarWait(my_s_ready + (kt & 1) * 8, (kt >> 1) & 1);
            if (!ok) {
                break;
            }
            tcgenFenceAfter();
            float s[kBN];
            tmemLoad64(tmem_s + lane_field, s);

            // ---- softmax of this thread's row (log2 domain) -------------------------------------------
            // "plain" tile (the same answer for every row of the CTA): no causal cut, no ragged end, no
            // ALiBi - the scale (> 0) folds into one fma per element and the row maximum can be taken on
            // the raw scores.
            const bool plain = (kv0 + kBN - 1 <= cache_len + t0) && (valid >= kBN) && (slope_log2 == 0.f) && (c_log2 > 0.f);
            float mx;
            if (plain) {
                mx = rowMax64(s) * c_log2;
            } else {
                mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < kBN; ++j) {
                    float x = s[j] * c_log2;
                    if (slope_log2 != 0.f) {
                        x += slope_log2 * static_cast<float>(kv0 + j - limit);
                    }
                    x = (kv0 + j <= limit && j < valid) ? x : -INFINITY;
                    s[j] = x; // already in the log2 domain
                    mx = fmaxf(mx, x);
                }
            }
            float alpha = 1.f;
            bool rescale = false;
            if (kt == 0) {
                m_used = (mx == -INFINITY) ? 0.f : mx; // nothing accumulated yet: no rescale needed
            } else if (mx > m_used + kLazyBits) {
                alpha = fastExp2(m_used - mx);
                m_used = mx;
                rescale = true;
            }
            // p_j = 2^(x_j - m); x_j = s_j * scale (plain) or s_j already transformed
            uint32_t pw[kBN / 2];
            float sum8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const float neg_m = -m_used;
            const float mul = plain ? c_log2 : 1.f; // transformed scores are already scaled
#pragma unroll
            for (int j = 0; j < kBN; j += 2) {
                float x0, x1;
                fma2(x0, x1, s[j], s[j + 1], mul, neg_m);
                const float p0 = fastExp2(x0);
                const float p1 = fastExp2(x1);
                add2(sum8[j & 6], sum8[(j & 6) + 1], p0, p1);
                pw[j / 2] = packPair(p0, p1, T());
            }
            l_run = l_run * alpha + (((sum8[0] + sum8[1]) + (sum8[2] + sum8[3])) + ((sum8[4] + sum8[5]) + (sum8[6] + sum8[7])));

            if (__any_sync(0xffffffffu, rescale)) {
                // O is about to be rescaled in place: the previous tile's P.V must have retired first.
                // (rescale implies kt > 0.)  warp-collective: every lane scales its own row, alpha = 1
                // where nothing changed.
                ok = mbarWait(my_o_done, (kt - 1) & 1);
                if (!ok) {
                    break;
                }
                tcgenFenceAfter();
#pragma unroll
                for (int c = 0; c < kHD / 32; ++c) {
                    float o[32];
                    tmemLoad32(tmem_o + lane_field + c * 32, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        o[i] *= alpha;
                    }
                    tmemStore32(tmem_o + lane_field + c * 32, o);
                }
            }
            if (valid < kBN) {
                // V rows past the end may hold anything: zero them so that 0 * garbage stays 0.  Every
                // q-tile's warps zero all of them (the tiles do not wait for one another).
                ok = mbarWait(v_full + stage * 8, (kt / kStages) & 1);
                if (!ok) {
                    break;
                }
                for (int idx = gtid; idx < (kBN - valid) * kChunks * 8; idx += 128) {
                    const int vrow = valid + idx / (kChunks * 8);
                    const int rest = idx % (kChunks * 8);
                    const uint32_t addr = v_tile + (rest / 8) * (kBN * 128) + vrow * 128 + (rest % 8) * 16;
                    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
                }
                // generic-proxy writes that the tensor core's async-proxy reads must see
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            // P goes where its scores came from: the first 32 columns of this tile's S buffer, two 16-bit
            // probabilities per column - the A operand of P.V, read by the tensor core straight from
            // tensor memory.  The other S buffer (P of the previous tile, perhaps still being read) is
            // not touched.  The store is ordered before the MMA by the fence and the barrier below.
            tmemStoreBits32(tmem_s + lane_field, pw);
            tcgenFenceBefore();
            __syncwarp();
            if (lane == 0) {
                mbarArrive(my_p_ready + (kt & 1) * 8);
            }
        }

        if (ok) {
            ok = mbarWait(my_o_done, (num_kv_tiles - 1) & 1);
        }
        if (!ok) {
            sh_failed = 1;
        }
        tcgenFenceAfter();
        const float inv = (ok && l_run > 0.f) ? 1.f / l_run : 0.f;
        // A tile whose 128 rows all belong to this sequence (or run past the end of the tensor, where
        // the store is clipped) leaves through shared memory - the Q tile's, free by now, in the same
        // swizzled layout - and one bulk tensor store per 64 columns: full lines instead of 16 bytes
        // per row per instruction.  A partial tile is written row by row.
        const bool bulk = a.tma_store != 0 && (rows_valid == kBM || q_begin + t0 + rows_valid == a.pp.total_q);
        T *out = static_cast<T *>(p.out) + (q_begin + t0 + row) * p.o_seq_stride + head * p.o_head_stride;
        const uint32_t o_stage = q_tiles + qi * kQBytes;
#pragma unroll
        for (int c = 0; c < kHD / 32; ++c) {
            float o[32];
            tmemLoad32(tmem_o + lane_field + c * 32, o); // warp-collective: rows past the chunk load too
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                uint4 v;
                v.x = packPair(o[i] * inv, o[i + 1] * inv, T());
                v.y = packPair(o[i + 2] * inv, o[i + 3] * inv, T());
                v.z = packPair(o[i + 4] * inv, o[i + 5] * inv, T());
                v.w = packPair(o[i + 6] * inv, o[i + 7] * inv, T());
                if (bulk) {
                    const int col = c * 32 + i; // 8 columns = one 16-byte piece of the 128-byte swizzled row
                    const uint32_t addr = o_stage + (col / 64) * (kBM * 128) + row * 128 + ((((col % 64) / 8) ^ (row & 7)) << 4);
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                } else if (ok && row < rows_valid) {
                    *reinterpret_cast<uint4 *>(out + c * 32 + i) = v;
                }
            }
        }
        if (bulk) {
            // every warp of the q-tile gets here (a failed wait only zeroes what it wrote)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync %0, 128;" ::"r"(1 + qi) : "memory");
            if ((warp & 3) == 0 && lane == 0 && sh_failed == 0) {
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    tmaStore3d(&tmap_o, o_stage + c * (kBM * 128), c * 64, head, static_cast<int>(q_begin + t0));
                }
                tmaStoreCommitAndWaitRead();
            }
        }
    }

    // ---- common exit: every role gets here on every path; TMEM reads and MMAs are done ------------
    tcgenFenceBefore();
    __syncthreads();
    if (threadIdx.x == 0 && sh_failed != 0 && p.kernel_flags != nullptr) {
        atomicOr(p.kernel_flags, 1u); // a bounded wait of this CTA ran out: its rows are missing (infiniopGetKernelStatus)
    }
    if (warp == kMmaWarp0) {
        tcgenFenceAfter();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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

CUtensorMapDataType mapDtype(infiniDtype_t dt) {
    return dt == INFINI_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
}

bool encodeCacheMap(CUtensorMap *map, const paged_attention::Info &A, const void *base, ptrdiff_t row_stride,
                    ptrdiff_t head_stride, ptrdiff_t block_stride, int box_rows) {
    EncodeTiledFn fn = encodeTiled();
    if (fn == nullptr) {
        return false;
    }
    const cuuint64_t dims[4] = {A.head_size, A.block_size, A.num_kv_heads, A.num_blocks};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(row_stride) * 2, static_cast<cuuint64_t>(head_stride) * 2,
                                   static_cast<cuuint64_t>(block_stride) * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    return fn(map, mapDtype(A.dtype), 4, const_cast<void *>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// q as {head_size, num_heads, total_q}: one box = 64 elements x 1 head x 128 tokens
bool encodeQueryMap(CUtensorMap *map, const Info &info, const void *base) {
    EncodeTiledFn fn = encodeTiled();
    if (fn == nullptr) {
        return false;
    }
    const auto &A = info.attn;
    const cuuint64_t dims[3] = {A.head_size, A.num_heads, info.total_q_tokens};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(A.q_head_stride) * 2, static_cast<cuuint64_t>(A.q_seq_stride) * 2};
    const cuuint32_t box[3] = {64, 1, kBM};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    return fn(map, mapDtype(A.dtype), 3, const_cast<void *>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// out as {head_size, num_heads, total_q}, same box as q; false when its strides do not fit a tensor map
bool encodeOutMap(CUtensorMap *map, const Info &info, const void *base) {
    EncodeTiledFn fn = encodeTiled();
    if (fn == nullptr) {
        return false;
    }
    const auto &A = info.attn;
    if (A.o_head_stride <= 0 || A.o_seq_stride <= 0 || (A.o_head_stride % 8) != 0 || (A.o_seq_stride % 8) != 0) {
        return false;
    }
    const cuuint64_t dims[3] = {A.head_size, A.num_heads, info.total_q_tokens};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(A.o_head_stride) * 2, static_cast<cuuint64_t>(A.o_seq_stride) * 2};
    const cuuint32_t box[3] = {64, 1, kBM};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    return fn(map, mapDtype(A.dtype), 3, const_cast<void *>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// tiles + barriers / TMEM slot / scan scratch
constexpr size_t smemBytes(int stages, int k_stages, int nq, int hd) {
    return static_cast<size_t>(nq) * qTileBytes(hd) + static_cast<size_t>(stages + k_stages) * kvTileBytes(hd) + 512;
}

template <typename T, int STAGES, int KSTAGES, int NQ, int HD>
infiniStatus_t launchTyped(const UmmaArgs &args, const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const CUtensorMap &mo,
                           unsigned tiles, int device_id, cudaStream_t stream) {
    static std::mutex attr_mutex;
    static bool attr_done[64] = {};
    auto kernel = pagedPrefillUmmaKernel<T, STAGES, KSTAGES, NQ, HD>;
    {
        std::lock_guard<std::mutex> lock(attr_mutex);
        const bool tracked = device_id >= 0 && device_id < 64;
        if (!tracked || !attr_done[device_id]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smemBytes(STAGES, KSTAGES, NQ, HD))) != cudaSuccess) {
                return checkLaunch("cudaFuncSetAttribute(pagedPrefillUmmaKernel)");
            }
            if (tracked) {
                attr_done[device_id] = true;
            }
        }
    }
    const dim3 grid(tiles, args.pp.d.num_heads / NQ);
    kernel<<<grid, 8 * NQ * 32, smemBytes(STAGES, KSTAGES, NQ, HD), stream>>>(mq, mk, mv, mo, args);
    return checkLaunch("pagedPrefillUmmaKernel");
}

template <typename T, int HD>
infiniStatus_t launchShape(int stages, int k_stages, int nq, const UmmaArgs &args, const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const CUtensorMap &mo,
                           unsigned tiles, int device_id, cudaStream_t stream) {
    if (nq == 2) {
        switch (stages) {
        case 2:
            return launchTyped<T, 2, 2, 2, HD>(args, mq, mk, mv, mo, tiles, device_id, stream);
        case 3:
            return launchTyped<T, 3, 3, 2, HD>(args, mq, mk, mv, mo, tiles, device_id, stream);
        default:
            return launchTyped<T, 4, 4, 2, HD>(args, mq, mk, mv, mo, tiles, device_id, stream);
        }
    }
    switch (stages) {
    case 2:
        return k_stages == 3 ? launchTyped<T, 2, 3, 1, HD>(args, mq, mk, mv, mo, tiles, device_id, stream)
                             : launchTyped<T, 2, 2, 1, HD>(args, mq, mk, mv, mo, tiles, device_id, stream);
    case 3:
        return launchTyped<T, 3, 3, 1, HD>(args, mq, mk, mv, mo, tiles, device_id, stream);
    default:
        return launchTyped<T, 4, 4, 1, HD>(args, mq, mk, mv, mo, tiles, device_id, stream);
    }
}

} // namespace

UmmaPlan planPrefillUmma(const Info &info, const DeviceProps &props) {
    UmmaPlan plan;
    const auto &A = info.attn;
    if ((A.head_size != 128 && A.head_size != 64) || A.value_size != A.head_size) {
        return plan;
    }
    if (A.block_size % 8 != 0 || A.num_seqs == 0 || A.num_seqs > 65536 || info.total_q_tokens == 0 || A.num_blocks == 0) {
        return plan;
    }
    // rows of one K/V copy: the largest of 64, 32, 16, 8 that divides the page, so a copy never crosses a page
    plan.box_rows = (A.block_size % 64 == 0) ? 64 : (A.block_size % 32 == 0) ? 32 : (A.block_size % 16 == 0) ? 16 : 8;
    auto mult8 = [](ptrdiff_t v) { return v > 0 && (v % 8) == 0; }; // 16 bytes of a 2-byte dtype
    if (!mult8(A.q_seq_stride) || !mult8(A.q_head_stride) || !mult8(A.o_seq_stride) || !mult8(A.o_head_stride)) {
        return plan;
    }
    if (!mult8(A.k_row_stride) || !mult8(A.k_head_stride) || !mult8(A.k_block_stride)
        || !mult8(A.v_row_stride) || !mult8(A.v_head_stride) || !mult8(A.v_block_stride)) {
        return plan;
    }
    CUtensorMap probe;
    void *fake = reinterpret_cast<void *>(static_cast<uintptr_t>(1) << 30);
    if (!encodeCacheMap(&probe, A, fake, A.k_row_stride, A.k_head_stride, A.k_block_stride, plan.box_rows)
        || !encodeCacheMap(&probe, A, fake, A.v_row_stride, A.v_head_stride, A.v_block_stride, plan.box_rows)
        || !encodeQueryMap(&probe, info, fake)) {
        return plan;
    }
    // One q-head per CTA, two CTAs per SM, measured fastest.  INFINIOP_PAGED_PREFILL_QTILES=2 (even GQA
    // groups only) lets the two q-heads of a pair share each staged KV tile in one CTA per SM instead:
    // half the L2 traffic for about 10% less throughput at the Llama-3-8B shape.
    const size_t group = A.num_heads / A.num_kv_heads;
    plan.q_tiles = 1;
    if (const char *env = std::getenv("INFINIOP_PAGED_PREFILL_QTILES")) {
        const int v = std::atoi(env);
        if (v == 1 || (v == 2 && group % 2 == 0)) {
            plan.q_tiles = v;
        }
    }
    // Two slots in the V ring and three in the K ring by default.  With two K slots the copy of a K tile
    // can only start when the scores two tiles earlier have retired and then lands about when its own scores
    // are wanted: cycle stamps of one CTA under load showed the softmax warps waiting ~1000 cycles for scores
    // every fourth or fifth tile.  The third K slot gives the copy a whole tile period of slack; the V tile
    // is wanted a tile later anyway.  32 KiB of Q + 3 x 16 + 2 x 16 KiB still lets two one-head CTAs share an
    // SM (head 128).  INFINIOP_PAGED_PREFILL_STAGES = 2..4 sets the V ring (and, from 3 up, both rings);
    // INFINIOP_PAGED_PREFILL_K_STAGES = 2 | 3 the K ring beside a two-slot V ring.
    plan.stages = 2;
    if (const char *env = std::getenv("INFINIOP_PAGED_PREFILL_STAGES")) {
        const int v = std::atoi(env);
        if (v >= 2 && v <= 4) {
            plan.stages = v;
        }
    }
    plan.k_stages = (plan.stages == 2 && plan.q_tiles == 1) ? 3 : plan.stages;
    if (const char *env = std::getenv("INFINIOP_PAGED_PREFILL_K_STAGES")) {
        const int v = std::atoi(env);
        if (plan.stages == 2 && plan.q_tiles == 1 && (v == 2 || v == 3)) {
            plan.k_stages = v;
        }
    }
    const int hd_i = static_cast<int>(A.head_size);
    while (plan.stages > 2 && smemBytes(plan.stages, plan.k_stages, plan.q_tiles, hd_i) > props.smem_per_block_optin) {
        --plan.stages;
        plan.k_stages = plan.stages;
    }
    if (smemBytes(plan.stages, plan.k_stages, plan.q_tiles, hd_i) > props.smem_per_block_optin) {
        return plan;
    }
    // INFINIOP_PAGED_PREFILL_TEST_DELAY_V_US (test only, at most 1000): the producers hold every V copy from the second
    // tile on back by that long, which puts the P.V issuer behind the softmax warps.
    if (const char *env = std::getenv("INFINIOP_PAGED_PREFILL_TEST_DELAY_V_US")) {
        const long long us = std::atoll(env);
        if (us >= 1 && us <= 1000) {
            plan.test_delay_v_cycles = us * 2000; // SM cycles at a nominal 2 GHz
        }
    }
    plan.eligible = true;
    return plan;
}

infiniStatus_t launchPrefillUmma(const Info &info, const UmmaPlan &plan, const PrefillParams &pp, cudaStream_t stream) {
    const auto &A = info.attn;
    const auto &p = pp.d;
    const auto addr = [](const void *ptr) { return reinterpret_cast<uintptr_t>(ptr); };
    if (((addr(p.k_cache) | addr(p.v_cache) | addr(p.q) | addr(p.out)) & 15u) != 0) {
        return launchPrefillGeneric(info, pp, stream);
    }
    CUtensorMap mq, mk, mv;
    B200_RETURN_IF(!encodeQueryMap(&mq, info, p.q), INFINI_STATUS_INTERNAL_ERROR);
    B200_RETURN_IF(!encodeCacheMap(&mk, A, p.k_cache, A.k_row_stride, A.k_head_stride, A.k_block_stride, plan.box_rows), INFINI_STATUS_INTERNAL_ERROR);
    B200_RETURN_IF(!encodeCacheMap(&mv, A, p.v_cache, A.v_row_stride, A.v_head_stride, A.v_block_stride, plan.box_rows), INFINI_STATUS_INTERNAL_ERROR);
    UmmaArgs args;
    args.pp = pp;
    args.box_rows = plan.box_rows;
    args.test_delay_v_cycles = plan.test_delay_v_cycles;
    CUtensorMap mo;
    args.tma_store = encodeOutMap(&mo, info, p.out) ? 1 : 0;
    if (!args.tma_store) {
        mo = mq; // never dereferenced
    }
    const unsigned tiles = static_cast<unsigned>((info.total_q_tokens + kBM - 1) / kBM + A.num_seqs);
    int device_id = -1;
    (void)cudaGetDevice(&device_id);
    if (A.head_size == 64) {
        return A.dtype == INFINI_DTYPE_F16 ? launchShape<__half, 64>(plan.stages, plan.k_stages, plan.q_tiles, args, mq, mk, mv, mo, tiles, device_id, stream)
                                           : launchShape<__nv_bfloat16, 64>(plan.stages, plan.k_stages, plan.q_tiles, args, mq, mk, mv, mo, tiles, device_id, stream);
    }
    return A.dtype == INFINI_DTYPE_F16 ? launchShape<__half, 128>(plan.stages, plan.k_stages, plan.q_tiles, args, mq, mk, mv, mo, tiles, device_id, stream)
                                       : launchShape<__nv_bfloat16, 128>(plan.stages, plan.k_stages, plan.q_tiles, args, mq, mk, mv, mo, tiles, device_id, stream);
}

} // namespace b200::paged_attention_prefill
