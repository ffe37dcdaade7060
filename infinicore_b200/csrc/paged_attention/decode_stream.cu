// Streaming paged-attention decode for sm_100a.
//
// What it computes is what the reference's split-KV decode computes
// (src/infiniop/ops/paged_attention/cuda/kernel_v2.cuh:620-1074 partial pass, :556-616
// combine): out[s,h,:] = softmax_t(scale * q[s,h,:] . K[s,t,kv(h),:]) . V[s,t,kv(h),:], fp32
// online softmax in the log2 domain.  How it gets there is different, and built around the
// one thing that bounds this op on a B200 - reading every K/V byte exactly once at HBM speed:
//
//  * Work decomposition.  A "tile" is 16 consecutive tokens of one KV page for one kv-head.
//    A "unit" is (sequence, kv-head, group of <= 8 q-heads that share that kv-head); its length
//    is ceil(seq_len / 16) tiles.  All units are laid end to end in one linear tile space and
//    that space is cut into equal contiguous ranges, one per persistent warp ("worker"), with no
//    host knowledge of seq_lens: the per-sequence tile prefix is built on the device.  A range is
//    cut once more, into "pieces": a head piece (its first 7/8) that the range's own worker streams,
//    and a few tail chunks of halving size that go into a pool shared by all workers.  A worker that
//    has finished takes the next chunk of the pool (one atomicAdd), so workers whose SM gets a
//    smaller share of the memory system - per-worker rates spread by about 3 % - hand the end of
//    their range to faster ones and everybody finishes together.  Piece boundaries depend only on
//    the lengths and the plan, never on timing, and every piece starts from fresh softmax state: the
//    result is bit-identical from run to run whoever computes a piece.
//  * Data movement.  Each worker owns a private ring of `stages` shared-memory slots.  Lanes
//    0..2*HD/64-1 each issue one non-multicast `cp.async.bulk.tensor` (TMA) box of
//    16 rows x 128 bytes with the 128-byte swizzle; completion is tracked by one mbarrier per
//    slot.  Block-table entries are fetched one tile ahead of the TMA issue that needs them, and the
//    next chunk is claimed one tile before the current piece runs out, so the ring never drains at
//    page, kv-head, sequence or piece boundaries.
//  * Arithmetic.  All q-heads of the GQA group consume the same staged tile:
//    S^T[8 heads x 16 tokens] = Q.K^T and O[8 heads x HD] += P.V run as warp-level
//    mma.sync.m16n8k16 (bf16/fp16 in, fp32 accumulate) with ldmatrix / ldmatrix.trans operand
//    loads that are bank-conflict-free under the swizzle.  P is rounded to the cache dtype
//    before the PV product, as the reference's torch check does
//    (test/infiniop/paged_attention.py:43).  Rows 8..15 of the M dimension are padding.
//  * Reduction.  A piece that covers a whole unit writes the normalised output directly.
//    Otherwise the worker writes (acc, m, l) to workspace slot (unit + piece): along the linear space
//    the pair (unit, piece) only ever moves forward in one or both coordinates, so that sum is
//    unique.  It then adds its tile count to the unit's counter (release fence, atomicAdd); whoever
//    brings the counter to the unit's length is the last to arrive and merges the unit's records in
//    piece order - nobody ever waits for anybody.  When a handful of very long sequences are cut into
//    hundreds of pieces each, a combine kernel (several CTAs per unit) merges instead.  A small
//    reset kernel in front clears the counters.  The only waits are mbarrier waits on a worker's own
//    TMA copies, and those are bounded.
//
// HBM traffic per launch: K and V tiles once each (the algorithmic bytes), plus q/out, block
// tables, and 8*(HD+2)*4 bytes written and read back per (unit, piece) boundary - at most
// units + pieces records.
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace b200::paged_attention {

namespace {

constexpr int kTileTokens = 16;
constexpr int kHeadsPerTile = 8;
constexpr int kMaxStages = 8;
constexpr int kMaxWarps = 8;
constexpr int kPlanThreads = 1024;
constexpr long long kWaitLimitCycles = 4000000000ll; // an mbarrier wait gives up after ~2 s
constexpr int kResetThreads = 1024;
constexpr int kMinDynamicRange = 32; // ranges shorter than this many tiles are not cut into pieces

struct PlanHeader {
    int reserved;
    int num_ranges; // ranges actually used (<= number of workers)
    long long total_tiles;
    long long range_len;
};

struct StreamArgs {
    DecodeParams p;
    PlanHeader *header;
    long long *prefix;  // [num_seqs + 1] tiles before each sequence (one kv-head, one head tile)
    int4 *range_start;  // [workers] (sequence, unit-within-sequence, tile) where a range begins
    int row_boxes;      // the tensor maps are the 5-D ones: one copy per tensor and tile
    int4 *tasks;        // [workers] combine tasks of the wide-head kernel: (sequence, unit-within-sequence, first range, records)
    int *counters;      // one-warp kernel: [0] next chunk of the pool, [1 + unit] tiles of the unit done so far; cleared by the reset kernel
    float *partials;    // [(units + pieces)] records of 8 * (HD + 2) floats
    int units_per_seq;  // num_kv_heads * head_tiles
    int head_tiles;
    int tiles_per_page; // block_size / 16
    int stages;
    int num_workers;
    int embedded_plan;   // 1: every CTA derives the plan itself in shared memory (no plan kernel)
    int max_chunks;      // tail chunks a range may be cut into (0: ranges are not cut)
    int min_chunk;       // smallest chunk, in tiles (the last chunk of a range takes what is left)
    int tail_shift;      // the last range_len >> tail_shift tiles of a range go to the pool
    int merge_in_kernel; // 1: the last worker to arrive at a unit merges its records; 0: the combine kernel does
    int l2_evict_first;  // 1: K/V copies carry the evict-first L2 policy
    long long wait_limit_cycles; // a bounded wait gives up after this many cycles of the SM's counter
    int withhold_first_copy;     // test only: worker 0 leaves out its first copy, so that its first wait runs out
};

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
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
__device__ __forceinline__ bool mbarWait(uint32_t bar, uint32_t parity, long long limit = kWaitLimitCycles) {
    if (mbarTryWait(bar, parity)) {
        return true;
    }
    const long long t0 = clock64();
    while (!mbarTryWait(bar, parity)) {
        if (clock64() - t0 > limit) {
            return false;
        }
    }
    return true;
}

// One TMA box {64 elements, 16 rows, 1 kv-head, 1 block} of a 4-D map
// {head_size, block_size, num_kv_heads, num_blocks} into swizzled shared memory.
__device__ __forceinline__ void tmaLoadBox(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                           int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// The same copy with an L2 eviction policy.  K and V are read once per launch: marked evict-first they
// leave the L2 to what IS read again - block tables, q rows and the split-unit records.
__device__ __forceinline__ void tmaLoadBoxHint(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                               int c0, int c1, int c2, int c3, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
        : "memory");
}

// One TMA box {64 elements, 16 rows, all 64-element column chunks, 1 kv-head, 1 block} of the 5-D map
// {64, block_size, width / 64, num_kv_heads, num_blocks}: the whole K (or V) part of a tile in one copy.  The
// chunk dimension's stride is 128 bytes - smaller than the row stride below it - so the box lands as
// [chunk][row][128 bytes], which is the layout the kernels read.  Issuing a copy holds the issuing warp for a
// couple of hundred cycles whatever its size, so one copy per tensor instead of one per chunk matters where a
// tile has many chunks (9 + 8 at key width 576).
__device__ __forceinline__ void tmaLoadRows(uint32_t dst, const CUtensorMap *map, uint32_t bar, int row0, int kv_head, int block) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(0), "r"(row0), "r"(0), "r"(kv_head), "r"(block)
        : "memory");
}
__device__ __forceinline__ void tmaLoadRowsHint(uint32_t dst, const CUtensorMap *map, uint32_t bar, int row0, int kv_head, int block,
                                                uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(0), "r"(row0), "r"(0), "r"(kv_head), "r"(block), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t evictFirstPolicy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ void ldmatrixX4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    // volatile keeps it after the (volatile) mbarrier wait; no memory clobber, so the compiler
    // may keep unrelated values in registers across it
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
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                        uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fastExp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream still runs; it must not touch global memory the
// predecessor may write until gridDependencyWait() returns (which is when the predecessor has
// completed and its writes are visible).  Every CTA executes the wait before it exits, so the
// ordering is transitive along a chain of such kernels.  Both are no-ops for a normal launch.
__device__ __forceinline__ void gridDependencyWait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void gridLaunchDependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint32_t packPair(float lo, float hi, __nv_bfloat16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t packPair(float lo, float hi, __half) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// ---------------------------------------------------------------------------------------
// Walking the linear tile space
// ---------------------------------------------------------------------------------------
struct Cursor {
    int s;   // sequence
    int j;   // unit within the sequence: kv_head * head_tiles + head_tile
    int ti;  // tile within the sequence
    int nt;  // tiles in sequence s
};

__device__ __forceinline__ void advance(Cursor &c, const long long *prefix, int num_seqs, int units_per_seq) {
    if (++c.ti == c.nt) {
        c.ti = 0;
        if (++c.j == units_per_seq) {
            c.j = 0;
            do {
                ++c.s;
                c.nt = (c.s < num_seqs) ? static_cast<int>(prefix[c.s + 1] - prefix[c.s]) : 1;
            } while (c.nt == 0);
        }
    }
}

// Where does linear position x start?  It belongs to the last sequence s with
// prefix[s] * units_per_seq <= x, i.e. prefix[s] <= x / units_per_seq.
__device__ __forceinline__ int4 locate(const long long *prefix, int num_seqs, int units_per_seq, long long x) {
    const long long y = x / units_per_seq;
    int lo = 0, hi = num_seqs; // invariant: prefix[lo] <= y < prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= y) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    const long long nt = prefix[lo + 1] - prefix[lo];
    const long long rem = x - prefix[lo] * units_per_seq;
    return make_int4(lo, static_cast<int>(rem / nt), static_cast<int>(rem % nt), 0);
}

// ---------------------------------------------------------------------------------------
// Pieces of a range
// ---------------------------------------------------------------------------------------
// Every range of `range_len` tiles is cut the same way: a head piece [0, range_len - budget) and
// `chunks` tail chunks that cover the last `budget` tiles; chunk i takes half of what is left (at
// least min_chunk tiles), the last possible chunk takes all of it.  Pieces are numbered along the
// tile space: range r owns ids r * (chunks + 1) + {0: head, 1 + i: chunk i}.
struct PieceGeometry {
    int budget;
    int chunks;
};

__device__ __forceinline__ int chunkLength(int rem, int index, int max_chunks, int min_chunk) {
    const int half = max((rem + 1) >> 1, min_chunk);
    return (index == max_chunks - 1) ? rem : min(half, rem);
}

__device__ __forceinline__ PieceGeometry pieceGeometry(long long range_len, int max_chunks, int min_chunk, int tail_shift) {
    PieceGeometry g;
    g.budget = 0;
    g.chunks = 0;
    if (max_chunks <= 0 || range_len < kMinDynamicRange || range_len > 0x3fffffffll) {
        return g;
    }
    g.budget = static_cast<int>(range_len >> tail_shift);
    int rem = g.budget;
    while (rem > 0 && g.chunks < max_chunks) {
        rem -= chunkLength(rem, g.chunks, max_chunks, min_chunk);
        ++g.chunks;
    }
    return g;
}

// Chunk j of a range: its first tile within the range and its length.
__device__ __forceinline__ void chunkSpan(long long range_len, PieceGeometry g, int max_chunks, int min_chunk, int j,
                                          int &begin, int &len) {
    int rem = g.budget;
    begin = static_cast<int>(range_len) - g.budget;
    len = 0;
    for (int i = 0; i <= j; ++i) {
        begin += len;
        len = chunkLength(rem, i, max_chunks, min_chunk);
        rem -= len;
    }
}

// Id of the piece that holds linear position x.
__device__ __forceinline__ long long pieceOf(long long x, long long range_len, PieceGeometry g, int max_chunks, int min_chunk) {
    // (positions and range lengths below 2^32 take the 32-bit division, several times cheaper than the 64-bit one)
    const long long r = ((x | range_len) >> 32) == 0 ? static_cast<long long>(static_cast<unsigned>(x) / static_cast<unsigned>(range_len))
                                                       : x / range_len;
    const long long id = r * (g.chunks + 1);
    if (g.chunks == 0) {
        return id;
    }
    const int off = static_cast<int>(x - r * range_len);
    int end = static_cast<int>(range_len) - g.budget; // end of the head piece
    if (off < end) {
        return id;
    }
    int rem = g.budget;
    for (int i = 0; i < g.chunks - 1; ++i) {
        const int len = chunkLength(rem, i, max_chunks, min_chunk);
        end += len;
        rem -= len;
        if (off < end) {
            return id + 1 + i;
        }
    }
    return id + g.chunks;
}

// ---------------------------------------------------------------------------------------
// Reset kernel: clears the chunk counter and the per-unit tile counters of the
// one-warp kernel.  It sits in front of every launch because the workspace is the caller's scratch:
// nothing can be assumed about what the previous user left in it.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kResetThreads)
    pagedDecodeResetKernel(const StreamArgs a, long long count) {
    gridDependencyWait(); // the previous launch on this workspace may still be counting
    gridLaunchDependents();
    for (long long i = static_cast<long long>(blockIdx.x) * kResetThreads + threadIdx.x; i < count;
         i += static_cast<long long>(gridDim.x) * kResetThreads) {
        a.counters[i] = 0;
    }
}

// ---------------------------------------------------------------------------------------
// Plan kernel: tile prefix per sequence, range length, and where each range starts.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kPlanThreads)
    pagedDecodePlanKernel(const StreamArgs a) {
    __shared__ long long warp_sums[kPlanThreads / 32];
    __shared__ long long running_s;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int wid = tid >> 5;
    const int num_seqs = a.p.num_seqs;
    const long long capacity = static_cast<long long>(a.p.max_blocks_per_seq) * a.p.block_size;

    gridDependencyWait();
    gridLaunchDependents();
    if (tid == 0) {
        running_s = 0;
        a.prefix[0] = 0;
    }
    __syncthreads();

    for (int base = 0; base < num_seqs; base += kPlanThreads) {
        const int s = base + tid;
        long long tiles = 0;
        if (s < num_seqs) {
            long long len = loadIndex(a.p.seq_lens, s, a.p.index_is_64);
            len = len < 0 ? 0 : (len > capacity ? capacity : len);
            tiles = (len + kTileTokens - 1) / kTileTokens;
        }
        long long incl = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) {
                incl += n;
            }
        }
        if (lane == 31) {
            warp_sums[wid] = incl;
        }
        __syncthreads();
        if (wid == 0) {
            long long v = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long n = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) {
                    v += n;
                }
            }
            warp_sums[lane] = v; // inclusive over warps
        }
        __syncthreads();
        const long long before = running_s + (wid > 0 ? warp_sums[wid - 1] : 0);
        if (s < num_seqs) {
            a.prefix[s + 1] = before + incl;
        }
        __syncthreads();
        if (tid == 0) {
            running_s += warp_sums[kPlanThreads / 32 - 1];
        }
        __syncthreads();
    }

    const long long seq_tiles = running_s;
    const long long total = seq_tiles * a.units_per_seq;
    long long range_len = (total + a.num_workers - 1) / a.num_workers;
    if (range_len < 1) {
        range_len = 1;
    }
    const int num_ranges = static_cast<int>((total + range_len - 1) / range_len);
    if (tid == 0) {
        a.header->num_ranges = num_ranges;
        a.header->total_tiles = total;
        a.header->range_len = range_len;
    }

    for (int r = tid; r < num_ranges; r += kPlanThreads) {
        a.range_start[r] = locate(a.prefix, num_seqs, a.units_per_seq, r * range_len);
    }
}

// ---------------------------------------------------------------------------------------
// Merge of a unit's records (one warp).  The records sit in consecutive slots, one per piece the
// unit touches, and are folded in that order - whichever worker arrived last and does it - so the
// result does not depend on timing.  Lane l handles float4 l, l + 32, ... of the HPT x HD accumulator
// block of a record; the (m, l) pairs follow the block.  Records are fetched a few at a time (all
// loads of a batch in flight together) and folded one after the other with the usual rescaling.
// Runs after the worker's streaming loop, when its registers are free; kept out of line.
// ---------------------------------------------------------------------------------------
constexpr int kMergeList = 20; // units a worker can note down for merging once its streaming is done
constexpr int kMergeStop = 8;  // ... and how many make it stop taking chunks from the pool

template <typename T, int HD, int HPT>
__device__ __noinline__ void mergeUnit(const StreamArgs &a, const long long *prefix, long long range_len, PieceGeometry geom,
                                       long long unit, int lane) {
    constexpr int kRec = HPT * (HD + 2);
    constexpr int kVecs = HPT * HD / 128;             // float4 per lane per record
    constexpr int kRowVecs = HD / 4;                  // float4 per accumulator row
    constexpr int kBatch = (32 / kVecs) > 0 ? (32 / kVecs) : 1; // records fetched together
    const DecodeParams &p = a.p;
    const int s = static_cast<int>(unit / a.units_per_seq);
    const int j = static_cast<int>(unit - static_cast<long long>(s) * a.units_per_seq);
    const long long nt = prefix[s + 1] - prefix[s];
    const long long xs = prefix[s] * a.units_per_seq + j * nt; // the unit's first tile in the linear space
    const long long p_first = pieceOf(xs, range_len, geom, a.max_chunks, a.min_chunk);
    const int nrec = static_cast<int>(pieceOf(xs + nt - 1, range_len, geom, a.max_chunks, a.min_chunk) - p_first) + 1;
    const int kv_head = j / a.head_tiles;
    const int head_tile = j % a.head_tiles;
    const int heads_valid = min(HPT, p.group_size - head_tile * HPT);
    const float *base = a.partials + (unit + p_first) * kRec;

    // (the caller has fenced: the other workers' records were published before they counted their tiles)
    float mx[kVecs], ls[kVecs];
    float4 acc[kVecs];
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
        mx[v] = -INFINITY;
        ls[v] = 0.f;
        acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int i0 = 0; i0 < nrec; i0 += kBatch) {
        float2 ml[kBatch][kVecs];
        float4 x[kBatch][kVecs];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            // past the last record: fetch the last one again, it is not folded
            const float *rr = base + static_cast<long long>(min(i0 + b, nrec - 1)) * kRec;
#pragma unroll
            for (int v = 0; v < kVecs; ++v) {
                const int f = v * 32 + lane;
                const int row = min(f / kRowVecs, heads_valid - 1);
                ml[b][v] = __ldcg(reinterpret_cast<const float2 *>(rr + HPT * HD + row * 2));
                x[b][v] = __ldcg(reinterpret_cast<const float4 *>(rr) + f);
            }
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            if (i0 + b < nrec) {
#pragma unroll
                for (int v = 0; v < kVecs; ++v) {
                    const float m_new = fmaxf(mx[v], ml[b][v].x);
                    const float keep = exp2f(mx[v] - m_new);
                    const float w = exp2f(ml[b][v].x - m_new);
                    acc[v].x = fmaf(w, x[b][v].x, acc[v].x * keep);
                    acc[v].y = fmaf(w, x[b][v].y, acc[v].y * keep);
                    acc[v].z = fmaf(w, x[b][v].z, acc[v].z * keep);
                    acc[v].w = fmaf(w, x[b][v].w, acc[v].w * keep);
                    ls[v] = fmaf(w, ml[b][v].y, ls[v] * keep);
                    mx[v] = m_new;
                }
            }
        }
    }
    const long long off0 = s * p.o_seq_stride + (kv_head * p.group_size + head_tile * HPT) * p.o_head_stride;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
        const int f = v * 32 + lane;
        const int row = f / kRowVecs;
        if (row < heads_valid) {
            const float inv = 1.f / ls[v];
            const long long off = off0 + row * p.o_head_stride + (f % kRowVecs) * 4;
            const uint32_t lo = packPair(acc[v].x * inv, acc[v].y * inv, T());
            const uint32_t hi = packPair(acc[v].z * inv, acc[v].w * inv, T());
            for (int d = 0; d <= p.num_extra_out; ++d) { // the output and every further destination
                T *out = static_cast<T *>(d == 0 ? p.out : p.extra_out[d - 1]) + off;
                *reinterpret_cast<uint32_t *>(out) = lo;
                *reinterpret_cast<uint32_t *>(out + 2) = hi;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Main kernel
// ---------------------------------------------------------------------------------------
// HPT: q-heads per head tile.  8 uses rows 0-7 of the MMA's M dimension (rows 8-15 are padding); 16 uses
// all rows, for groups of more than 8 q-heads per kv-head: K/V are then re-read once per 16 heads.
// Head 64 wants three resident CTAs per SM (half the bytes per tile, the same per-tile latencies): its
// CTAs are bounded to four warps so that the register allocation leaves room for three.
// POOL: ranges are cut into pieces and their tail chunks claimed from the pool (otherwise that code is not compiled in).
template <typename T, int HD, int HPT, bool POOL>
__global__ void __launch_bounds__(HD == 64 ? 128 : kMaxWarps * 32, HD == 64 ? 3 : 1)
    pagedDecodeStreamKernel(const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v,
                            const __grid_constant__ StreamArgs a) {
    constexpr int kChunks = HD / 64;               // 128-byte column chunks per row
    constexpr int kBoxBytes = kTileTokens * 128;   // one TMA box
    constexpr int kTensorBytes = kChunks * kBoxBytes;
    constexpr int kStageBytes = 2 * kTensorBytes;  // K tile + V tile
    constexpr int kKSteps = HD / 16;
    constexpr int kNTiles = HD / 8;
    constexpr int kRows = HPT / 8; // q-heads per thread: MMA rows g (and g + 8)
    static_assert(HPT == 8 || HPT == 16, "8 or 16 q-heads per head tile");

    extern __shared__ __align__(1024) unsigned char smem_raw[];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2; // MMA row (q-head within the head tile) / B-fragment column
    const int t = lane & 3;
    const int nwarps = blockDim.x >> 5;
    const int stages = a.stages;
    const DecodeParams &p = a.p;

    const uint32_t ring = smemAddr(smem_raw) + warp * stages * kStageBytes;
    const uint32_t bars = smemAddr(smem_raw) + nwarps * stages * kStageBytes + warp * stages * 8;
    // units this worker merges once its streaming is done
    long long *merge_list = reinterpret_cast<long long *>(smem_raw + nwarps * stages * (kStageBytes + 8)) + warp * kMergeList;
    // shared-memory copy of the plan (embedded mode): tile prefix per sequence + scan scratch
    long long *prefix_s = reinterpret_cast<long long *>(smem_raw + nwarps * stages * (kStageBytes + 8)) + nwarps * kMergeList;
    long long *scan_s = prefix_s + (p.num_seqs + 1);

    if (lane == 0) {
        for (int i = 0; i < stages; ++i) {
            mbarInit(bars + i * 8, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // The two tensor maps are kernel parameters: fetching them into the copy engine's descriptor cache does
    // not read anything an earlier kernel may still be writing.
    if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_v)) : "memory");
    }
    // Everything above touches only this CTA's shared memory; from here on global memory that an
    // earlier kernel in the stream may have produced is read.
    gridDependencyWait();
    gridLaunchDependents();

    const int worker = blockIdx.x * nwarps + warp;
    const long long *prefix;
    long long total_tiles, range_len;
    int num_ranges;
    if (a.embedded_plan) {
        // Every CTA derives the same plan: per-thread chunk of sequences -> block scan -> prefix.
        const int tid = threadIdx.x;
        const int nthreads = blockDim.x;
        const int per = (p.num_seqs + nthreads - 1) / nthreads;
        const long long capacity = static_cast<long long>(p.max_blocks_per_seq) * p.block_size;
        const int s_begin = min(tid * per, p.num_seqs);
        const int s_end = min(s_begin + per, p.num_seqs);
        long long mine = 0;
        for (int s = s_begin; s < s_end; ++s) {
            long long len = loadIndex(p.seq_lens, s, p.index_is_64);
            len = len < 0 ? 0 : (len > capacity ? capacity : len);
            mine += (len + kTileTokens - 1) / kTileTokens;
        }
        long long incl = mine;
#pragma unroll
        for (int o2 = 1; o2 < 32; o2 <<= 1) {
            const long long n = __shfl_up_sync(0xffffffffu, incl, o2);
            if (lane >= o2) {
                incl += n;
            }
        }
        if (lane == 31) {
            scan_s[warp] = incl;
        }
        __syncthreads();
        long long before = incl - mine;
        for (int w = 0; w < warp; ++w) {
            before += scan_s[w];
        }
        for (int s = s_begin; s < s_end; ++s) {
            long long len = loadIndex(p.seq_lens, s, p.index_is_64);
            len = len < 0 ? 0 : (len > capacity ? capacity : len);
            before += (len + kTileTokens - 1) / kTileTokens;
            prefix_s[s + 1] = before;
        }
        if (tid == 0) {
            prefix_s[0] = 0;
        }
        __syncthreads();
        prefix = prefix_s;
        total_tiles = prefix_s[p.num_seqs] * a.units_per_seq;
        range_len = (total_tiles + a.num_workers - 1) / a.num_workers;
        range_len = range_len < 1 ? 1 : range_len;
        num_ranges = static_cast<int>((total_tiles + range_len - 1) / range_len);
        if (blockIdx.x == 0) {
            // the combine kernel reads the plan from the workspace
            for (int s = tid; s <= p.num_seqs; s += nthreads) {
                a.prefix[s] = prefix_s[s];
            }
            if (tid == 0) {
                a.header->num_ranges = num_ranges;
                a.header->total_tiles = total_tiles;
                a.header->range_len = range_len;
            }
        }
    } else {
        prefix = a.prefix;
        total_tiles = a.header->total_tiles;
        range_len = a.header->range_len;
        num_ranges = a.header->num_ranges;
    }
    if (worker >= num_ranges) {
        return;
    }
    // The range's pieces: this worker streams the head piece, then chunks of the pool.
    const PieceGeometry geom = pieceGeometry(range_len, POOL ? a.max_chunks : 0, a.min_chunk, a.tail_shift);
    const int pieces_per_range = geom.chunks + 1;
    const int pool_total = num_ranges * geom.chunks;
    const long long x0 = worker * range_len;

    const int4 rs = a.embedded_plan ? locate(prefix, p.num_seqs, a.units_per_seq, x0) : a.range_start[worker];
    Cursor gen; // next tile to fetch
    gen.s = rs.x;
    gen.j = rs.y;
    gen.ti = rs.z;
    gen.nt = static_cast<int>(prefix[rs.x + 1] - prefix[rs.x]);
    Cursor cur = gen; // next tile to consume

    // Consumer side: the piece whose tiles are being consumed.  Generator side: the piece whose tiles
    // are being fetched - the same one (g_same) or, once that is fully issued, the next one (q_*).
    // (a range holds fewer than 2^31 tiles: the plan refuses shapes where it could hold more)
    const long long head_tiles_left = (total_tiles - x0 < range_len - geom.budget) ? (total_tiles - x0) : (range_len - geom.budget);
    int c_left = static_cast<int>(head_tiles_left); // tiles of the piece still to consume
    int c_id = worker * pieces_per_range;
    int g_left = c_left; // tiles of the generator's piece still to issue
    bool g_same = true;
    Cursor q_start = gen;
    int q_id = 0;
    int q_count = 0;
    bool pool_empty = (pool_total == 0);
    bool stop_claiming = false; // this worker has noted enough units to merge: it takes no further chunk
    bool ahead = false; // lane 0 holds a claimed pool index in k_ahead
    int k_ahead = 0;
    int free_slots = stages;
    int gen_stage = 0;

    const int tpp = a.tiles_per_page;
    const int head_tiles = a.head_tiles;
    const uint64_t stream_policy = evictFirstPolicy();

    bool withhold = a.withhold_first_copy != 0 && worker == 0;
    auto tableEntry = [&](const Cursor &c) -> long long {
        const int page = (tpp == 1) ? c.ti : c.ti / tpp;
        return reportedBlock(p, loadIndex(p.block_tables, c.s * p.bt_seq_stride + page, p.index_is_64));
    };
    auto issue = [&](int stage, const Cursor &c, long long block) {
        const uint32_t bar = bars + stage * 8;
        const uint32_t dst = ring + stage * kStageBytes;
        if (lane == 0) {
            mbarExpectTx(bar, kStageBytes);
        }
        const bool skip = withhold && lane == 0; // test only: the bytes are expected and never arrive
        withhold = false;
        if (a.row_boxes) {
            if (lane < 2 && !skip) {
                const int row0 = (tpp == 1) ? 0 : (c.ti % tpp) * kTileTokens;
                const int kv_head = (head_tiles == 1) ? c.j : c.j / head_tiles;
                if (a.l2_evict_first) {
                    tmaLoadRowsHint(dst + lane * kTensorBytes, lane ? &tmap_v : &tmap_k, bar, row0, kv_head, static_cast<int>(block), stream_policy);
                } else {
                    tmaLoadRows(dst + lane * kTensorBytes, lane ? &tmap_v : &tmap_k, bar, row0, kv_head, static_cast<int>(block));
                }
            }
        } else if (lane < 2 * kChunks && !skip) {
            const int is_v = lane / kChunks;
            const int chunk = lane % kChunks;
            const int row0 = (tpp == 1) ? 0 : (c.ti % tpp) * kTileTokens;
            const int kv_head = (head_tiles == 1) ? c.j : c.j / head_tiles;
            if (a.l2_evict_first) {
                tmaLoadBoxHint(dst + is_v * kTensorBytes + chunk * kBoxBytes, is_v ? &tmap_v : &tmap_k, bar,
                               chunk * 64, row0, kv_head, static_cast<int>(block), stream_policy);
            } else {
                tmaLoadBox(dst + is_v * kTensorBytes + chunk * kBoxBytes, is_v ? &tmap_v : &tmap_k, bar,
                           chunk * 64, row0, kv_head, static_cast<int>(block));
            }
        }
    };
    auto claim = [&]() -> int { // the pool index lands in lane 0
        int k = 0;
        if (lane == 0) {
            k = atomicAdd(a.counters, 1);
        }
        return k;
    };
    long long next_block = tableEntry(gen); // table entry of the generator's tile, fetched ahead of its issue

    // Issues the generator's next tile into the next free slot.  False when there is nothing to issue:
    // the pool is empty (or this worker claims no more), or the generator has finished the piece after the
    // consumer's and may not open a third.  (Every claimed chunk is processed: `ahead` is only ever dropped
    // by using k_ahead.)
    auto tryIssue = [&]() -> bool {
        if (g_left == 0) {
            if (!POOL || !g_same) {
                return false;
            }
            for (;;) {
                if (!ahead && (pool_empty || stop_claiming)) {
                    return false;
                }
                int k = ahead ? k_ahead : claim();
                ahead = false;
                k = __shfl_sync(0xffffffffu, k, 0);
                if (k >= pool_total) {
                    pool_empty = true;
                    return false;
                }
                // the pool hands out every range's first (largest) chunk before any second one
                const int j = k / num_ranges;
                const int r = k - j * num_ranges;
                int begin, len;
                chunkSpan(range_len, geom, a.max_chunks, a.min_chunk, j, begin, len);
                const long long qx0 = r * range_len + begin;
                const long long avail = total_tiles - qx0;
                if (avail <= 0) {
                    continue; // the last range is shorter than the others
                }
                q_count = avail < len ? static_cast<int>(avail) : len;
                q_id = r * pieces_per_range + 1 + j;
                const int4 qs = locate(prefix, p.num_seqs, a.units_per_seq, qx0);
                gen.s = qs.x;
                gen.j = qs.y;
                gen.ti = qs.z;
                gen.nt = static_cast<int>(prefix[qs.x + 1] - prefix[qs.x]);
                q_start = gen;
                g_left = q_count;
                g_same = false;
                next_block = tableEntry(gen);
                break;
            }
        }
        issue(gen_stage, gen, next_block);
        gen_stage = (gen_stage + 1 == stages) ? 0 : gen_stage + 1;
        --free_slots;
        --g_left;
        if (g_left > 0) {
            advance(gen, prefix, p.num_seqs, a.units_per_seq);
            next_block = tableEntry(gen);
        }
        if (POOL && g_left == 1 && !ahead && !pool_empty && !stop_claiming) {
            // one tile before the piece runs out: the atomic's round trip hides behind that tile
            k_ahead = claim();
            ahead = true;
        }
        return true;
    };
    auto refill = [&]() {
        while (free_slots > 0 && tryIssue()) {
        }
    };

    // ---- prologue: fill the ring ------------------------------------------------------
    refill();

    // ---- per-unit state ---------------------------------------------------------------
    uint32_t qa[kKSteps][2 * kRows]; // [.][2h], [.][2h + 1]: low / high 8 of the k-step, q-head g + 8h
    float o[kNTiles][4];
    float m_run[kRows], l_run[kRows], slope_log2[kRows];
    bool row_valid[kRows];
    int first_ti = cur.ti;
    int seq_len = 0;

    auto loadUnit = [&]() {
        const int kv_head = cur.j / head_tiles;
        const int head_tile = cur.j % head_tiles;
#pragma unroll
        for (int h = 0; h < kRows; ++h) {
            const int head_in_group = head_tile * HPT + g + 8 * h;
            row_valid[h] = head_in_group < p.group_size;
            const int head = kv_head * p.group_size + (row_valid[h] ? head_in_group : 0);
            const T *q = static_cast<const T *>(p.q) + cur.s * p.q_seq_stride + head * p.q_head_stride;
#pragma unroll
            for (int ks = 0; ks < kKSteps; ++ks) {
                qa[ks][2 * h] = row_valid[h] ? *reinterpret_cast<const uint32_t *>(q + ks * 16 + 2 * t) : 0u;
                qa[ks][2 * h + 1] = row_valid[h] ? *reinterpret_cast<const uint32_t *>(q + ks * 16 + 8 + 2 * t) : 0u;
            }
            slope_log2[h] = (p.alibi_slopes != nullptr && row_valid[h]) ? p.alibi_slopes[head] * 1.4426950408889634f : 0.f;
            m_run[h] = -INFINITY;
            l_run[h] = 0.f;
        }
        long long len = loadIndex(p.seq_lens, cur.s, p.index_is_64);
        const long long capacity = static_cast<long long>(p.max_blocks_per_seq) * p.block_size;
        seq_len = static_cast<int>(len > capacity ? capacity : len);
#pragma unroll
        for (int n = 0; n < kNTiles; ++n) {
            o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        }
        first_ti = cur.ti;
    };
    loadUnit();

    // ---- split units: who merges ----------------------------------------------------------
    // A record is published in two lazy steps, so that nothing here waits on the memory system in the
    // middle of the stream.  When the NEXT record is about to be written (or the stream is over): a fence
    // - the record's stores were issued a piece ago and have long landed - and an atomicAdd of the
    // segment's tile count on the unit's counter, whose return value stays in flight.  One step later that
    // value is looked at: the worker that brought the count to the unit's length is the last to arrive, every
    // other record of the unit is visible to it, and it notes the unit down; it merges its noted units when
    // its streaming is done.  Nobody waits for anybody.
    bool pend_valid = false, infl_valid = false;
    long long pend_unit = 0, infl_unit = 0;
    int pend_tiles = 0, pend_nt = 0, infl_tiles = 0, infl_nt = 0, infl_before = 0;
    int merge_count = 0;
    auto countSegments = [&]() {
        if (infl_valid) {
            const int before = __shfl_sync(0xffffffffu, infl_before, 0);
            if (before + infl_tiles == infl_nt) {
                if (lane == 0) {
                    merge_list[merge_count] = infl_unit;
                }
                // With kMergeStop units noted the worker claims no further chunk.  What it still holds - the
                // piece it consumes, the one after and a chunk claimed ahead, two partial segments each, plus
                // the two segments in the counting steps - adds at most eight, so the list never overflows.
                if (++merge_count >= kMergeStop) {
                    stop_claiming = true;
                }
            }
            infl_valid = false;
        }
        if (pend_valid) {
            __threadfence();
            __syncwarp();
            if (lane == 0) {
                infl_before = atomicAdd(a.counters + 1 + pend_unit, pend_tiles);
            }
            infl_unit = pend_unit;
            infl_tiles = pend_tiles;
            infl_nt = pend_nt;
            infl_valid = true;
            pend_valid = false;
        }
    };

    bool failed = false;
    int stage = 0;
    uint32_t parity = 0;

    for (;;) {
        const uint32_t bar = bars + stage * 8;
        const uint32_t k_tile = ring + stage * kStageBytes;
        const uint32_t v_tile = k_tile + kTensorBytes;
        if (!mbarWait(bar, parity, a.wait_limit_cycles)) {
            failed = true;
            break;
        }

        {
        const int tok0 = cur.ti * kTileTokens;
        const int valid = seq_len - tok0; // >= 1 by construction
        if (p.new_k != nullptr && valid <= kTileTokens) {
            // Decode step with append: this is the tile that holds the sequence's newest position
            // (row valid - 1).  Its K and V come from the caller's new rows, not from what the cache
            // held when the tile was fetched: overwrite the row in shared memory (same swizzle as the
            // copy engine's) and, once per (sequence, kv-head), store it into the cache for later steps.
            constexpr int kPieces = HD / 8; // 16-byte pieces per row
            const int kv_head = cur.j / head_tiles;
            const int row = valid - 1;
            const T *nk = static_cast<const T *>(p.new_k) + cur.s * p.new_k_seq_stride + kv_head * HD;
            const T *nv = static_cast<const T *>(p.new_v) + cur.s * p.new_v_seq_stride + kv_head * HD;
            bool writer = (cur.j % head_tiles) == 0;
            const long long block = writer ? tableEntry(cur) : 0;
            if (static_cast<unsigned long long>(block) >= static_cast<unsigned long long>(p.num_blocks)) {
                writer = false; // a table entry outside the pool: the row is used for this step but not stored
            }
            const int row_in_block = (seq_len - 1) % p.block_size;
            T *kc = static_cast<T *>(const_cast<void *>(p.k_cache)) + block * p.k_block_stride + kv_head * p.k_head_stride + row_in_block * p.k_row_stride;
            T *vc = static_cast<T *>(const_cast<void *>(p.v_cache)) + block * p.v_block_stride + kv_head * p.v_head_stride + row_in_block * p.v_row_stride;
            for (int idx = lane; idx < 2 * kPieces; idx += 32) {
                const int is_v = idx / kPieces;
                const int piece = idx % kPieces;
                const uint4 val = *reinterpret_cast<const uint4 *>((is_v ? nv : nk) + piece * 8);
                const uint32_t addr = (is_v ? v_tile : k_tile) + (piece >> 3) * kBoxBytes + row * 128 + (((piece & 7) ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w) : "memory");
                if (writer) {
                    *reinterpret_cast<uint4 *>((is_v ? vc : kc) + piece * 8) = val;
                }
            }
            // these generic-proxy writes precede the next TMA write into the same slot
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }
        if (valid < kTileTokens) {
            // Rows past the end of the sequence may hold anything (including NaN bit patterns):
            // K rows are neutralised by the -inf mask below, V rows must be zeroed because
            // 0 * NaN would poison the accumulators.
            for (int idx = lane; idx < (kTileTokens - valid) * kChunks * 8; idx += 32) {
                const int row = valid + idx / (kChunks * 8);
                const int rest = idx % (kChunks * 8);
                const uint32_t addr = v_tile + (rest / 8) * kBoxBytes + row * 128 + (rest % 8) * 16;
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
            }
            // these generic-proxy writes precede the next TMA write into the same slot
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }

        // Operand loads are issued ahead of the math that needs them: all K fragments, then (for
        // head sizes up to 128) all V fragments, so their shared-memory latency overlaps the QK
        // MMAs and the softmax instead of sitting in front of every MMA.
        const int k_row = ((lane >> 4) << 3) + (lane & 7);     // token row this lane addresses for K
        const int k_half = (lane >> 3) & 1;                     // which 16-byte column of the 32-byte k-step
        const int v_row = (((lane >> 3) & 1) << 3) + (lane & 7);
        const int v_sel = lane >> 4;
        auto kAddr = [&](int ks) {
            const int col = ks * 2 + k_half;
            return k_tile + (col >> 3) * kBoxBytes + k_row * 128 + (((col & 7) ^ (k_row & 7)) << 4);
        };
        auto vAddr = [&](int np) {
            const int col = np * 2 + v_sel;
            return v_tile + (col >> 3) * kBoxBytes + v_row * 128 + (((col & 7) ^ (v_row & 7)) << 4);
        };
        constexpr int kKChunk = (kKSteps <= 8) ? kKSteps : ((kKSteps % 8 == 0) ? 8 : 6); // divides kKSteps, even
        constexpr bool kPrefetchV = (HD <= 128);
        constexpr int kVFrags = kPrefetchV ? kNTiles / 2 : 1;

        // ---- S^T = Q . K^T: two accumulator chains per 8-token n-tile -----------------------
        float sa[2][4], sb[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            sa[n][0] = sa[n][1] = sa[n][2] = sa[n][3] = 0.f;
            sb[n][0] = sb[n][1] = sb[n][2] = sb[n][3] = 0.f;
        }
        uint32_t vb[kVFrags][4];
#pragma unroll
        for (int c0 = 0; c0 < kKSteps; c0 += kKChunk) {
            uint32_t kb[kKChunk][4];
#pragma unroll
            for (int ks = 0; ks < kKChunk; ++ks) {
                ldmatrixX4(kAddr(c0 + ks), kb[ks][0], kb[ks][1], kb[ks][2], kb[ks][3]);
            }
            if constexpr (kPrefetchV) {
                if (c0 == 0) {
#pragma unroll
                for (int np = 0; np < kVFrags; ++np) {
                    ldmatrixX4Trans(vAddr(np), vb[np][0], vb[np][1], vb[np][2], vb[np][3]);
                }
                }
            }
#pragma unroll
            for (int ks = 0; ks < kKChunk; ks += 2) {
                // A fragment: (row g, k low), (row g + 8, k low), (row g, k high), (row g + 8, k high)
                const uint32_t a1 = (kRows == 2) ? qa[c0 + ks][2 * (kRows - 1)] : 0u;
                const uint32_t a3 = (kRows == 2) ? qa[c0 + ks][2 * (kRows - 1) + 1] : 0u;
                const uint32_t b1 = (kRows == 2) ? qa[c0 + ks + 1][2 * (kRows - 1)] : 0u;
                const uint32_t b3 = (kRows == 2) ? qa[c0 + ks + 1][2 * (kRows - 1) + 1] : 0u;
                mma16816<T>(sa[0], qa[c0 + ks][0], a1, qa[c0 + ks][1], a3, kb[ks][0], kb[ks][1]);
                mma16816<T>(sa[1], qa[c0 + ks][0], a1, qa[c0 + ks][1], a3, kb[ks][2], kb[ks][3]);
                mma16816<T>(sb[0], qa[c0 + ks + 1][0], b1, qa[c0 + ks + 1][1], b3, kb[ks + 1][0], kb[ks + 1][1]);
                mma16816<T>(sb[1], qa[c0 + ks + 1][0], b1, qa[c0 + ks + 1][1], b3, kb[ks + 1][2], kb[ks + 1][3]);
            }
        }

        // ---- online softmax (log2 domain) for q-head g (and g + 8) over this tile's 16 tokens -----
        uint32_t pa[4] = {0u, 0u, 0u, 0u}; // A fragment of P: (row g | g + 8) x (tokens 2t, 2t+1 | 2t+8, 2t+9)
        float alpha[kRows];
#pragma unroll
        for (int h = 0; h < kRows; ++h) {
            float x[4];
            x[0] = (sa[0][2 * h] + sb[0][2 * h]) * p.scale_log2e;
            x[1] = (sa[0][2 * h + 1] + sb[0][2 * h + 1]) * p.scale_log2e;
            x[2] = (sa[1][2 * h] + sb[1][2 * h]) * p.scale_log2e;
            x[3] = (sa[1][2 * h + 1] + sb[1][2 * h + 1]) * p.scale_log2e;
            if (slope_log2[h] != 0.f) {
                const int rel = tok0 + 2 * t - (seq_len - 1);
                x[0] += slope_log2[h] * static_cast<float>(rel);
                x[1] += slope_log2[h] * static_cast<float>(rel + 1);
                x[2] += slope_log2[h] * static_cast<float>(rel + 8);
                x[3] += slope_log2[h] * static_cast<float>(rel + 9);
            }
            if (valid < kTileTokens) {
                const int c = 2 * t;
                x[0] = (c < valid) ? x[0] : -INFINITY;
                x[1] = (c + 1 < valid) ? x[1] : -INFINITY;
                x[2] = (c + 8 < valid) ? x[2] : -INFINITY;
                x[3] = (c + 9 < valid) ? x[3] : -INFINITY;
            }
            float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[h], mx);
            alpha[h] = fastExp2(m_run[h] - m_new);
            const float p0 = fastExp2(x[0] - m_new);
            const float p1 = fastExp2(x[1] - m_new);
            const float p2 = fastExp2(x[2] - m_new);
            const float p3 = fastExp2(x[3] - m_new);
            l_run[h] = l_run[h] * alpha[h] + ((p0 + p1) + (p2 + p3));
            m_run[h] = m_new;
            pa[h] = packPair(p0, p1, T());
            pa[2 + h] = packPair(p2, p3, T());
        }
#pragma unroll
        for (int n = 0; n < kNTiles; ++n) {
            o[n][0] *= alpha[0];
            o[n][1] *= alpha[0];
            if (kRows == 2) {
                o[n][2] *= alpha[kRows - 1];
                o[n][3] *= alpha[kRows - 1];
            }
        }

        // ---- O += P . V -----------------------------------------------------------------
#pragma unroll
        for (int np = 0; np < kNTiles / 2; ++np) {
            uint32_t b0, b1, b2, b3;
            if constexpr (kPrefetchV) {
                b0 = vb[np][0];
                b1 = vb[np][1];
                b2 = vb[np][2];
                b3 = vb[np][3];
            } else {
                ldmatrixX4Trans(vAddr(np), b0, b1, b2, b3);
            }
            mma16816<T>(o[2 * np], pa[0], pa[1], pa[2], pa[3], b0, b1);
            mma16816<T>(o[2 * np + 1], pa[0], pa[1], pa[2], pa[3], b2, b3);
        }

        }

        // ---- the slot is free: top the ring up (this may open the next piece) --------------------
        __syncwarp();
        ++free_slots;
        if (++stage == stages) {
            stage = 0;
            parity ^= 1u;
        }
        refill();
        --c_left;

        // ---- end of unit or end of piece: emit --------------------------------------------
        const bool unit_end = (cur.ti + 1 == cur.nt);
        if (unit_end || c_left == 0) {
            const int kv_head = cur.j / head_tiles;
            const int head_tile = cur.j % head_tiles;
            const long long unit = static_cast<long long>(cur.s) * a.units_per_seq + cur.j;
            const bool whole_unit = (first_ti == 0 && unit_end);
            float *rec = a.partials + (unit + c_id) * (HPT * (HD + 2));
            if (!whole_unit && a.merge_in_kernel) {
                countSegments(); // before this record's stores: the fence in there is about the previous record
            }
#pragma unroll
            for (int h = 0; h < kRows; ++h) {
                float l_all = l_run[h];
                l_all += __shfl_xor_sync(0xffffffffu, l_all, 1);
                l_all += __shfl_xor_sync(0xffffffffu, l_all, 2);
                const int r = g + 8 * h;
                if (whole_unit) {
                    if (row_valid[h]) {
                        const int head = kv_head * p.group_size + head_tile * HPT + r;
                        const long long off = cur.s * p.o_seq_stride + head * p.o_head_stride;
                        const float inv = 1.f / l_all;
                        for (int d = 0; d <= p.num_extra_out; ++d) { // the output and every further destination
                            T *out = static_cast<T *>(d == 0 ? p.out : p.extra_out[d - 1]) + off;
#pragma unroll
                            for (int n = 0; n < kNTiles; ++n) {
                                *reinterpret_cast<uint32_t *>(out + n * 8 + 2 * t) = packPair(o[n][2 * h] * inv, o[n][2 * h + 1] * inv, T());
                            }
                        }
                    }
                } else {
                    if (row_valid[h]) {
#pragma unroll
                        for (int n = 0; n < kNTiles; ++n) {
                            *reinterpret_cast<float2 *>(rec + r * HD + n * 8 + 2 * t) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
                        }
                    }
                    if (t == 0 && row_valid[h]) {
                        *reinterpret_cast<float2 *>(rec + HPT * HD + r * 2) = make_float2(m_run[h], l_all);
                    }
                }
            }
            if (!whole_unit && a.merge_in_kernel) {
                pend_unit = unit;
                pend_tiles = cur.ti - first_ti + 1;
                pend_nt = cur.nt;
                pend_valid = true;
            }
        }
        if (c_left > 0) {
            advance(cur, prefix, p.num_seqs, a.units_per_seq);
            if (unit_end) {
                loadUnit();
            }
        } else {
            // The piece is done.  refill() above has already tried to open the next one.
            if (g_same) {
                break;
            }
            cur = q_start;
            c_left = q_count;
            c_id = q_id;
            g_same = true;
            loadUnit();
        }
    }

    if (!failed && a.merge_in_kernel) {
        // The stream is over: count the last segment first (its fence and the atomic's round trip then
        // overlap the look at the count that is still in flight), note what this worker arrived last at,
        // and merge.
        int before_last = 0;
        if (pend_valid) {
            __threadfence();
            __syncwarp();
            if (lane == 0) {
                before_last = atomicAdd(a.counters + 1 + pend_unit, pend_tiles);
            }
        }
        const bool had_pending = pend_valid;
        pend_valid = false;
        countSegments(); // looks at the count in flight
        if (had_pending) {
            before_last = __shfl_sync(0xffffffffu, before_last, 0);
            if (before_last + pend_tiles == pend_nt) {
                if (lane == 0) {
                    merge_list[merge_count] = pend_unit;
                }
                ++merge_count;
            }
        }
        __syncwarp();
        if (merge_count > 0) {
            __threadfence(); // the other workers' records were published before they counted their tiles
        }
        for (int i = 0; i < merge_count; ++i) {
            mergeUnit<T, HD, HPT>(a, prefix, range_len, geom, merge_list[i], lane);
        }
    }

    if (failed) {
        if (lane == 0 && p.kernel_flags != nullptr) {
            atomicOr(p.kernel_flags, 1u);
        }
        // Let this worker's copies still in flight land (bounded) before its shared memory is
        // released: they sit in slots `stage`, `stage + 1`, ... in issue order.
        int sidx = stage;
        uint32_t par = parity;
        for (int k = free_slots; k < stages; ++k) {
            (void)mbarWait(bars + sidx * 8, par, a.wait_limit_cycles);
            if (++sidx == stages) {
                sidx = 0;
                par ^= 1u;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Wide-head kernel: key width 576 (value width 576, or 512 for latent attention).
//
// Same decomposition, plan, partial records and combine as above, with two differences.
//  * One worker is a CTA of four warps instead of one warp: a 16-token tile is 36 KiB here and the O
//    accumulator of a head tile does not fit one warp's registers.  The four warps share one ring of
//    staged tiles.  Each warp multiplies a quarter of the key width (9 of the 36 k-steps) for the
//    scores S^T = Q.K^T of the tile, the four partial sums meet in shared memory (1 KiB per warp, two
//    buffers so that one CTA-wide barrier per tile is enough) and every warp adds them in the same
//    order, so the four hold identical scores and identical softmax state; each owns a quarter of the
//    value columns for O += P.V.  (Every warp computing all 36 k-steps itself needs no barrier but
//    2.6 times the tensor-core and ldmatrix instructions per tile, and the kernel is bound by those, not
//    by HBM.)  A tile is two copies (5-D tensor maps: all column chunks of the K part, of the V part), issued by
//    warps 0 and 1; with the 4-D maps it is 17 or 18 copies shared out over the four warps.  Every warp arrives
//    on the slot's barrier for the bytes it asked for.  A slot is handed back through an "empty" mbarrier on which each of the four warps
//    arrives once it has read the slot; before they consume tile i, the warps refill the slot tile
//    i - 1 has just left.
//  * A head tile is 16 q-heads, all 16 rows of the MMA's M dimension: shapes with many q-heads per
//    kv-head (latent attention: 128) re-read K/V once per 16 heads instead of once per 8.  The unit's Q
//    rows live in shared memory (16 x 576 values, padded rows) and reach the MMA through ldmatrix.
// All waits are bounded.  A wait that runs out does not leave the loop: the warp keeps walking it
// with its work switched off, so the four warps reach every CTA-wide barrier together.
// ---------------------------------------------------------------------------------------
constexpr int kWideWarps = 4;
constexpr int kWideHeads = 16;
#ifndef B200_WIDE_DEFAULT_STAGES
#define B200_WIDE_DEFAULT_STAGES 3
#endif
constexpr int kWideDefaultStages = B200_WIDE_DEFAULT_STAGES; // ring slots per CTA unless the environment says otherwise

template <typename T, int KD, int VD>
__global__ void __launch_bounds__(kWideWarps * 32)
    pagedDecodeWideKernel(const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v,
                          const StreamArgs a) {
    constexpr int kKChunks = KD / 64;
    constexpr int kVChunks = VD / 64;
    constexpr int kBoxBytes = kTileTokens * 128;
    constexpr int kKBytes = kKChunks * kBoxBytes;
    constexpr int kVBytes = kVChunks * kBoxBytes;
    constexpr int kStageBytes = kKBytes + kVBytes;
    constexpr int kKSteps = KD / 16;
    constexpr int kWarpKSteps = kKSteps / kWideWarps; // k-steps of the scores each warp multiplies: 9
    constexpr int kKChunk = 3;                        // k-steps fetched per batch of ldmatrix (divides 9)
    constexpr int kPartialBytes = kWideHeads * kTileTokens * 4; // one warp's partial scores: 1 KiB
    constexpr int kCols = VD / kWideWarps;            // value columns per warp: 144 or 128
    constexpr int kNTiles = kCols / 8;                // 18 or 16 (even)
    constexpr int kVPieces = kCols / 8;               // 16-byte pieces of a V row per warp
    constexpr int kQStride = KD * 2 + 16;             // bytes per Q row in shared memory: odd multiple of 16 -> conflict-free ldmatrix
    constexpr int kQBytes = kWideHeads * kQStride;
    static_assert(kKSteps % kWideWarps == 0 && kWarpKSteps % kKChunk == 0 && kNTiles % 2 == 0 && kKChunks + kVChunks <= 32, "shape");

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int stages = a.stages;
    const DecodeParams &p = a.p;

    const uint32_t ring = smemAddr(smem_raw);
    const uint32_t q_smem = ring + stages * kStageBytes;
    const uint32_t full = q_smem + kQBytes;
    const uint32_t empty = full + stages * 8;
    const uint32_t partials = empty + stages * 8; // [2 buffers][4 warps][1 KiB]; 16-byte aligned (every term is)
    unsigned char *q_ptr = smem_raw + stages * kStageBytes;

    if (threadIdx.x == 0) {
        for (int i = 0; i < stages; ++i) {
            mbarInit(full + i * 8, kWideWarps);
            mbarInit(empty + i * 8, kWideWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    gridDependencyWait();
    gridLaunchDependents();

    const int worker = blockIdx.x;
    const long long *prefix = a.prefix;
    const long long total_tiles = a.header->total_tiles;
    const long long range_len = a.header->range_len;
    const int num_ranges = a.header->num_ranges;
    if (worker >= num_ranges) {
        return;
    }
    const long long x0 = worker * range_len;
    const long long count = (total_tiles - x0 < range_len) ? (total_tiles - x0) : range_len;
    const int4 rs = a.range_start[worker];
    Cursor gen;
    gen.s = rs.x;
    gen.j = rs.y;
    gen.ti = rs.z;
    gen.nt = static_cast<int>(prefix[rs.x + 1] - prefix[rs.x]);
    Cursor cur = gen;

    if (threadIdx.x == 0) {
        int4 task = make_int4(-1, -1, 0, 0);
        if (rs.z != 0) {
            const long long unit_start = x0 - rs.z;
            const long long r_first = unit_start / range_len;
            if (worker == r_first + 1) {
                const long long r_last = (unit_start + gen.nt - 1) / range_len;
                task = make_int4(rs.x, rs.y, static_cast<int>(r_first), static_cast<int>(r_last - r_first + 1));
            }
        }
        a.tasks[worker] = task;
    }

    const int tpp = a.tiles_per_page;
    const int head_tiles = a.head_tiles;
    auto tableEntry = [&](const Cursor &c) -> long long {
        const int page = (tpp == 1) ? c.ti : c.ti / tpp;
        return reportedBlock(p, loadIndex(p.block_tables, c.s * p.bt_seq_stride + page, p.index_is_64));
    };
    // The copies of a tile are shared out over the four warps (a copy costs its issuing lane on the
    // order of a hundred cycles, and the lanes of one warp issue one after another): warp w takes
    // boxes w, w + 4, ... of the K chunks followed by the V chunks, one box per lane, and announces
    // its own bytes with its own arrival on the slot's barrier.
    constexpr int kBoxes = kKChunks + kVChunks;
    const uint64_t stream_policy = evictFirstPolicy();
    const int my_box = warp + kWideWarps * lane;
    const bool has_box = my_box < kBoxes;
    // (with the 5-D maps: warp 0 copies the K part of a tile, warp 1 the V part, the other two only arrive)
    const uint32_t my_bytes = a.row_boxes ? (warp == 0 ? kKBytes : warp == 1 ? kVBytes : 0u)
                                          : static_cast<uint32_t>((kBoxes - warp + kWideWarps - 1) / kWideWarps) * kBoxBytes;
    auto issue = [&](int stage, const Cursor &c, long long block) {
        const uint32_t bar = full + stage * 8;
        const uint32_t dst = ring + stage * kStageBytes;
        if (lane == 0) {
            mbarExpectTx(bar, my_bytes);
        }
        __syncwarp();
        if (a.row_boxes) {
            if (warp < 2 && lane == 0) {
                const int row0 = (tpp == 1) ? 0 : (c.ti % tpp) * kTileTokens;
                const int kv_head = (head_tiles == 1) ? c.j : c.j / head_tiles;
                if (a.l2_evict_first) {
                    tmaLoadRowsHint(dst + (warp ? kKBytes : 0), warp ? &tmap_v : &tmap_k, bar, row0, kv_head, static_cast<int>(block), stream_policy);
                } else {
                    tmaLoadRows(dst + (warp ? kKBytes : 0), warp ? &tmap_v : &tmap_k, bar, row0, kv_head, static_cast<int>(block));
                }
            }
        } else if (has_box) {
            const int is_v = my_box >= kKChunks;
            const int chunk = is_v ? my_box - kKChunks : my_box;
            const int row0 = (tpp == 1) ? 0 : (c.ti % tpp) * kTileTokens;
            const int kv_head = (head_tiles == 1) ? c.j : c.j / head_tiles;
            if (a.l2_evict_first) {
                tmaLoadBoxHint(dst + (is_v ? kKBytes : 0) + chunk * kBoxBytes, is_v ? &tmap_v : &tmap_k, bar,
                               chunk * 64, row0, kv_head, static_cast<int>(block), stream_policy);
            } else {
                tmaLoadBox(dst + (is_v ? kKBytes : 0) + chunk * kBoxBytes, is_v ? &tmap_v : &tmap_k, bar,
                           chunk * 64, row0, kv_head, static_cast<int>(block));
            }
        }
    };

    long long issued = 0;
    for (int i = 0; i < stages && i < count; ++i) {
        issue(i, gen, tableEntry(gen));
        ++issued;
        if (issued < count) {
            advance(gen, prefix, p.num_seqs, a.units_per_seq);
        }
    }
    long long next_block = (issued < count) ? tableEntry(gen) : 0;

    // ---- per-unit state: two q-heads per thread (MMA rows g and g + 8) ------------------------
    float o[kNTiles][4];
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    float slope_log2[2] = {0.f, 0.f};
    bool row_valid[2] = {false, false};
    int first_ti = cur.ti, seq_len = 0;
    // CTA-wide: the four warps copy the unit's 16 Q rows (zero rows past the group) into shared memory
    auto loadUnit = [&]() {
        const int kv_head = cur.j / head_tiles;
        const int head_tile = cur.j % head_tiles;
        constexpr int kPiecesPerRow = KD / 8;
        for (int idx = threadIdx.x; idx < kWideHeads * kPiecesPerRow; idx += kWideWarps * 32) {
            const int r = idx / kPiecesPerRow;
            const int piece = idx % kPiecesPerRow;
            const int head_in_group = head_tile * kWideHeads + r;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (head_in_group < p.group_size) {
                const T *q = static_cast<const T *>(p.q) + cur.s * p.q_seq_stride + (kv_head * p.group_size + head_in_group) * p.q_head_stride;
                val = *reinterpret_cast<const uint4 *>(q + piece * 8);
            }
            *reinterpret_cast<uint4 *>(q_ptr + r * kQStride + piece * 16) = val;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int head_in_group = head_tile * kWideHeads + g + 8 * h;
            row_valid[h] = head_in_group < p.group_size;
            const int head = kv_head * p.group_size + (row_valid[h] ? head_in_group : 0);
            slope_log2[h] = (p.alibi_slopes != nullptr && row_valid[h]) ? p.alibi_slopes[head] * 1.4426950408889634f : 0.f;
            m_run[h] = -INFINITY;
            l_run[h] = 0.f;
        }
        long long len = loadIndex(p.seq_lens, cur.s, p.index_is_64);
        const long long capacity = static_cast<long long>(p.max_blocks_per_seq) * p.block_size;
        seq_len = static_cast<int>(len > capacity ? capacity : len);
#pragma unroll
        for (int n = 0; n < kNTiles; ++n) {
            o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        }
        first_ti = cur.ti;
    };
    loadUnit();
    __syncthreads();

    bool failed = false;
    int stage = 0;
    uint32_t parity = 0;
    for (long long i = 0; i < count; ++i) {
        const uint32_t k_tile = ring + stage * kStageBytes;
        const uint32_t v_tile = k_tile + kKBytes;
        // first refill the slot of the previous tile (the four warps have just left it) with tile
        // i - 1 + stages, so that stages - 1 tiles are in flight behind the one being consumed
        if (!failed && i >= 1 && issued < count) {
            const int prev_stage = (stage == 0) ? stages - 1 : stage - 1;
            const uint32_t prev_parity = (stage == 0) ? (parity ^ 1u) : parity; // phase of the slot's latest use
            if (!mbarWait(empty + prev_stage * 8, prev_parity)) {
                failed = true;
            } else {
                issue(prev_stage, gen, next_block);
                ++issued;
                if (issued < count) {
                    advance(gen, prefix, p.num_seqs, a.units_per_seq);
                    next_block = tableEntry(gen);
                }
            }
        }
        if (!failed && !mbarWait(full + stage * 8, parity)) {
            failed = true;
        }
        const int tok0 = cur.ti * kTileTokens;
        const int valid = seq_len - tok0; // >= 1 by construction
        const int v_piece0 = warp * kVPieces; // this warp's first 16-byte piece of a V row
        const int k_row = ((lane >> 4) << 3) + (lane & 7);
        const int k_half = (lane >> 3) & 1;
        const int v_row = (((lane >> 3) & 1) << 3) + (lane & 7);
        const int v_sel = lane >> 4;
        auto kAddr = [&](int ks) {
            const int col = ks * 2 + k_half;
            return k_tile + (col >> 3) * kBoxBytes + k_row * 128 + (((col & 7) ^ (k_row & 7)) << 4);
        };
        auto vAddr = [&](int np) { // np counts pairs of 8-column n-tiles inside this warp's slice
            const int col = v_piece0 + np * 2 + v_sel;
            return v_tile + (col >> 3) * kBoxBytes + v_row * 128 + (((col & 7) ^ (v_row & 7)) << 4);
        };
        // A fragment of k-step ks: matrices (rows 0-7 | 8-15) x (columns 16 ks .. +8 | +8 .. +16)
        const uint32_t q_lane = q_smem + ((lane & 7) + ((lane >> 3) & 1) * 8) * kQStride + (lane >> 4) * 16;

        float sa[2][4], sb[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            sa[n][0] = sa[n][1] = sa[n][2] = sa[n][3] = 0.f;
            sb[n][0] = sb[n][1] = sb[n][2] = sb[n][3] = 0.f;
        }

        if (!failed) {
        if (p.new_k != nullptr && valid <= kTileTokens) {
            // Decode step with append: every warp swaps the newest row into what it reads itself (all of
            // K, its own value columns); the stores into the cache are shared out the same way.
            constexpr int kKPieces = KD / 8;
            const int kv_head = cur.j / head_tiles;
            const int row = valid - 1;
            const T *nk = static_cast<const T *>(p.new_k) + cur.s * p.new_k_seq_stride + kv_head * KD;
            const T *nv = static_cast<const T *>(p.new_v) + cur.s * p.new_v_seq_stride + kv_head * VD;
            bool writer = (cur.j % head_tiles) == 0;
            const long long block = writer ? tableEntry(cur) : 0;
            if (static_cast<unsigned long long>(block) >= static_cast<unsigned long long>(p.num_blocks)) {
                writer = false; // a table entry outside the pool: the row is used for this step but not stored
            }
            const int row_in_block = (seq_len - 1) % p.block_size;
            T *kc = static_cast<T *>(const_cast<void *>(p.k_cache)) + block * p.k_block_stride + kv_head * p.k_head_stride + row_in_block * p.k_row_stride;
            T *vc = static_cast<T *>(const_cast<void *>(p.v_cache)) + block * p.v_block_stride + kv_head * p.v_head_stride + row_in_block * p.v_row_stride;
            for (int piece = lane; piece < kKPieces; piece += 32) {
                const uint4 val = *reinterpret_cast<const uint4 *>(nk + piece * 8);
                const uint32_t addr = k_tile + (piece >> 3) * kBoxBytes + row * 128 + (((piece & 7) ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w) : "memory");
                if (writer && warp == 0) {
                    *reinterpret_cast<uint4 *>(kc + piece * 8) = val;
                }
            }
            for (int q8 = lane; q8 < kVPieces; q8 += 32) {
                const int piece = v_piece0 + q8;
                const uint4 val = *reinterpret_cast<const uint4 *>(nv + piece * 8);
                const uint32_t addr = v_tile + (piece >> 3) * kBoxBytes + row * 128 + (((piece & 7) ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w) : "memory");
                if (writer) {
                    *reinterpret_cast<uint4 *>(vc + piece * 8) = val;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }
        if (valid < kTileTokens) {
            // V rows past the end may hold anything: zero this warp's columns of them (0 * NaN would
            // poison the accumulators); K rows are neutralised by the -inf mask below.
            for (int idx = lane; idx < (kTileTokens - valid) * kVPieces; idx += 32) {
                const int row = valid + idx / kVPieces;
                const int piece = v_piece0 + idx % kVPieces;
                const uint32_t addr = v_tile + (piece >> 3) * kBoxBytes + row * 128 + (((piece & 7) ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }

        // ---- S^T = Q . K^T, 16 heads x 16 tokens: this warp's quarter of the key width ---------------
        const int ks0 = warp * kWarpKSteps;
#pragma unroll
        for (int c0 = 0; c0 < kWarpKSteps; c0 += kKChunk) {
            uint32_t kb[kKChunk][4], qf[kKChunk][4];
#pragma unroll
            for (int ks = 0; ks < kKChunk; ++ks) {
                ldmatrixX4(kAddr(ks0 + c0 + ks), kb[ks][0], kb[ks][1], kb[ks][2], kb[ks][3]);
                ldmatrixX4(q_lane + (ks0 + c0 + ks) * 32, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
            }
#pragma unroll
            for (int ks = 0; ks < kKChunk; ++ks) {
                // two independent accumulator chains, alternating
                if (((c0 + ks) & 1) == 0) {
                    mma16816<T>(sa[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kb[ks][0], kb[ks][1]);
                    mma16816<T>(sa[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kb[ks][2], kb[ks][3]);
                } else {
                    mma16816<T>(sb[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kb[ks][0], kb[ks][1]);
                    mma16816<T>(sb[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kb[ks][2], kb[ks][3]);
                }
            }
        }
        } // !failed
        // ---- the four partial sums meet: every warp of the CTA takes part in the barrier on every tile,
        // also one whose wait ran out (its scores are then meaningless; the status word says so) ----------
        {
            const uint32_t mine = partials + ((static_cast<uint32_t>(i) & 1u) * kWideWarps + warp) * kPartialBytes + lane * 32;
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(mine), "f"(sa[0][0] + sb[0][0]), "f"(sa[0][1] + sb[0][1]),
                         "f"(sa[0][2] + sb[0][2]), "f"(sa[0][3] + sb[0][3]) : "memory");
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(mine + 16), "f"(sa[1][0] + sb[1][0]), "f"(sa[1][1] + sb[1][1]),
                         "f"(sa[1][2] + sb[1][2]), "f"(sa[1][3] + sb[1][3]) : "memory");
            asm volatile("bar.sync 1, %0;" ::"n"(kWideWarps * 32) : "memory");
            float part[kWideWarps][8];
#pragma unroll
            for (int w = 0; w < kWideWarps; ++w) {
                const uint32_t src = partials + ((static_cast<uint32_t>(i) & 1u) * kWideWarps + w) * kPartialBytes + lane * 32;
                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(part[w][0]), "=f"(part[w][1]), "=f"(part[w][2]), "=f"(part[w][3]) : "r"(src) : "memory");
                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(part[w][4]), "=f"(part[w][5]), "=f"(part[w][6]), "=f"(part[w][7]) : "r"(src + 16) : "memory");
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                sa[0][e] = (part[0][e] + part[1][e]) + (part[2][e] + part[3][e]);
                sa[1][e] = (part[0][4 + e] + part[1][4 + e]) + (part[2][4 + e] + part[3][4 + e]);
            }
        }
        if (!failed) {

        // ---- online softmax (log2 domain) of rows g and g + 8, identical in the four warps ----------
        uint32_t pa[4]; // A fragment of P: (row g | g + 8) x (tokens 2t, 2t+1 | 2t+8, 2t+9)
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float x[4];
            x[0] = sa[0][2 * h] * p.scale_log2e;
            x[1] = sa[0][2 * h + 1] * p.scale_log2e;
            x[2] = sa[1][2 * h] * p.scale_log2e;
            x[3] = sa[1][2 * h + 1] * p.scale_log2e;
            if (slope_log2[h] != 0.f) {
                const int rel = tok0 + 2 * t - (seq_len - 1);
                x[0] += slope_log2[h] * static_cast<float>(rel);
                x[1] += slope_log2[h] * static_cast<float>(rel + 1);
                x[2] += slope_log2[h] * static_cast<float>(rel + 8);
                x[3] += slope_log2[h] * static_cast<float>(rel + 9);
            }
            if (valid < kTileTokens) {
                const int c = 2 * t;
                x[0] = (c < valid) ? x[0] : -INFINITY;
                x[1] = (c + 1 < valid) ? x[1] : -INFINITY;
                x[2] = (c + 8 < valid) ? x[2] : -INFINITY;
                x[3] = (c + 9 < valid) ? x[3] : -INFINITY;
            }
            float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[h], mx);
            alpha[h] = fastExp2(m_run[h] - m_new);
            const float p0 = fastExp2(x[0] - m_new);
            const float p1 = fastExp2(x[1] - m_new);
            const float p2 = fastExp2(x[2] - m_new);
            const float p3 = fastExp2(x[3] - m_new);
            l_run[h] = l_run[h] * alpha[h] + ((p0 + p1) + (p2 + p3));
            m_run[h] = m_new;
            pa[h] = packPair(p0, p1, T());
            pa[2 + h] = packPair(p2, p3, T());
        }
#pragma unroll
        for (int n = 0; n < kNTiles; ++n) {
            o[n][0] *= alpha[0];
            o[n][1] *= alpha[0];
            o[n][2] *= alpha[1];
            o[n][3] *= alpha[1];
        }

        // ---- O += P . V over this warp's value columns ------------------------------------------
#pragma unroll
        for (int np = 0; np < kNTiles / 2; ++np) {
            uint32_t b0, b1, b2, b3;
            ldmatrixX4Trans(vAddr(np), b0, b1, b2, b3);
            mma16816<T>(o[2 * np], pa[0], pa[1], pa[2], pa[3], b0, b1);
            mma16816<T>(o[2 * np + 1], pa[0], pa[1], pa[2], pa[3], b2, b3);
        }

        // ---- this warp is done with the slot ---------------------------------------------------------
        __syncwarp();
        if (lane == 0) {
            mbarArrive(empty + stage * 8);
        }
        } // !failed

        if (++stage == stages) {
            stage = 0;
            parity ^= 1u;
        }

        // ---- end of unit or end of range: emit ------------------------------------------------------
        const bool unit_end = (cur.ti + 1 == cur.nt);
        if ((unit_end || i + 1 == count) && !failed) {
            const int kv_head = cur.j / head_tiles;
            const int head_tile = cur.j % head_tiles;
            const int col0 = warp * kCols; // this warp's first value column
            const long long unit = static_cast<long long>(cur.s) * a.units_per_seq + cur.j;
            float *rec = a.partials + (unit + worker) * (kWideHeads * (VD + 2));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float l_all = l_run[h];
                l_all += __shfl_xor_sync(0xffffffffu, l_all, 1);
                l_all += __shfl_xor_sync(0xffffffffu, l_all, 2);
                const int r = g + 8 * h;
                if (first_ti == 0 && unit_end) {
                    if (row_valid[h]) {
                        const int head = kv_head * p.group_size + head_tile * kWideHeads + r;
                        const long long off = cur.s * p.o_seq_stride + head * p.o_head_stride + col0;
                        const float inv = 1.f / l_all;
                        for (int d = 0; d <= p.num_extra_out; ++d) { // the output and every further destination
                            T *out = static_cast<T *>(d == 0 ? p.out : p.extra_out[d - 1]) + off;
#pragma unroll
                            for (int n = 0; n < kNTiles; ++n) {
                                *reinterpret_cast<uint32_t *>(out + n * 8 + 2 * t) = packPair(o[n][2 * h] * inv, o[n][2 * h + 1] * inv, T());
                            }
                        }
                    }
                } else if (row_valid[h]) {
#pragma unroll
                    for (int n = 0; n < kNTiles; ++n) {
                        *reinterpret_cast<float2 *>(rec + r * VD + col0 + n * 8 + 2 * t) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
                    }
                    if (warp == 0 && t == 0) {
                        *reinterpret_cast<float2 *>(rec + kWideHeads * VD + r * 2) = make_float2(m_run[h], l_all);
                    }
                }
            }
        }
        if (i + 1 < count) {
            advance(cur, prefix, p.num_seqs, a.units_per_seq);
            if (unit_end) {
                __syncthreads(); // every warp has read the old unit's Q rows for the last time
                loadUnit();
                __syncthreads();
            }
        }
    }

    if (failed && lane == 0 && p.kernel_flags != nullptr) {
        atomicOr(p.kernel_flags, 1u);
    }
    // Copies still in flight must land before the CTA's shared memory is released.  A warp whose
    // wait ran out drains its own slots: whichever phase is pending, a bounded wait on both
    // parities covers it.
    if (failed) {
        for (int sidx = 0; sidx < stages; ++sidx) {
            (void)mbarWait(full + sidx * 8, 0);
            (void)mbarWait(full + sidx * 8, 1);
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------
// Combine kernel.  A unit is split exactly when a range boundary falls inside it, so there are
// fewer split units than workers.  The worker whose range starts at the FIRST boundary inside a
// unit leaves a task (sequence, unit, first range, number of records) in tasks[worker]; CTA r of
// this kernel executes tasks[r].  Its warps share out the unit's records, each warp merges its
// share with a warp-local running maximum, and the per-warp results are merged through shared
// memory - the same (m, l, acc) algebra at both levels.
// ---------------------------------------------------------------------------------------
// A record holds 8 heads x VD accumulator floats, then 8 x (m, l).  One CTA merges the columns
// [blockIdx.y * HD, +HD) of a unit's records: HD = VD for the widths one CTA can hold, 64 for the
// wide-head kernel (grid.y = VD / 64).
template <int HD, int VD, int HPT>
struct CombineShape {
    static constexpr int kWarps = (HD <= 128) ? 8 : 4;
    static constexpr int kFloats = HPT * HD;                  // accumulator floats per record slice
    static constexpr int kVec = kFloats / 4 / 32;             // float4 per lane per record slice
    static constexpr int kRec = HPT * (VD + 2);
    static constexpr int kMl = HPT * VD;                      // offset of the (m, l) pairs in a record
};

// HPT: q-heads per head tile (8 or 16 for the one-warp kernel, 16 for the wide-head kernel).
// BY_UNIT: CTA x merges unit x and finds the unit's records from the plan (one-warp kernel, used when a
// few very long units are cut into many pieces each); otherwise CTA x executes tasks[x] (wide-head kernel).
template <typename T, int HD, int VD = HD, int HPT = kHeadsPerTile, bool BY_UNIT = false>
__global__ void __launch_bounds__(CombineShape<HD, VD, HPT>::kWarps * 32)
    pagedDecodeCombineKernel(const StreamArgs a) {
    using S = CombineShape<HD, VD, HPT>;
    __shared__ float4 acc_s[S::kWarps][S::kFloats / 4];
    __shared__ float m_s[S::kWarps][HPT];
    __shared__ float l_s[S::kWarps][HPT];

    const DecodeParams &p = a.p;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    gridDependencyWait(); // records, plan, tasks and directly written `out` rows come from the main kernel
    gridLaunchDependents();
    int s, j, n;
    long long first_piece;
    if constexpr (BY_UNIT) {
        s = static_cast<int>(blockIdx.x / a.units_per_seq);
        j = static_cast<int>(blockIdx.x % a.units_per_seq);
        const long long nt = a.prefix[s + 1] - a.prefix[s];
        if (nt == 0) {
            return;
        }
        const long long range_len = a.header->range_len;
        const PieceGeometry geom = pieceGeometry(range_len, a.max_chunks, a.min_chunk, a.tail_shift);
        const long long xs = a.prefix[s] * a.units_per_seq + j * nt;
        first_piece = pieceOf(xs, range_len, geom, a.max_chunks, a.min_chunk);
        n = static_cast<int>(pieceOf(xs + nt - 1, range_len, geom, a.max_chunks, a.min_chunk) - first_piece) + 1;
        if (n == 1) {
            return; // one piece covered the unit and wrote `out` itself
        }
    } else {
        const int r = blockIdx.x;
        if (r >= a.header->num_ranges) {
            return;
        }
        const int4 task = a.tasks[r];
        n = task.w;
        if (n <= 0) {
            return;
        }
        s = task.x;
        j = task.y;
        first_piece = task.z;
    }
    const int kv_head = j / a.head_tiles;
    const int head_tile = j % a.head_tiles;
    const int heads_valid = min(HPT, p.group_size - head_tile * HPT);
    const long long unit = static_cast<long long>(s) * a.units_per_seq + j;
    const float *base = a.partials + (unit + first_piece) * S::kRec;
    const int slice0 = static_cast<int>(blockIdx.y) * HD; // first value column this CTA merges

    // vector v of this lane covers floats [4 * (v * 32 + lane), +4) of the record slice: head
    // (v * 32 + lane) / (HD / 4), columns slice0 + 4 * ((v * 32 + lane) % (HD / 4)) ...
    int head_of[S::kVec];
    float m_loc[S::kVec], l_loc[S::kVec];
    float4 acc[S::kVec];
#pragma unroll
    for (int v = 0; v < S::kVec; ++v) {
        head_of[v] = (v * 32 + lane) / (HD / 4);
        m_loc[v] = -INFINITY;
        l_loc[v] = 0.f;
        acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int i = warp; i < n; i += S::kWarps) {
        const float *ml = base + static_cast<long long>(i) * S::kRec + S::kMl;
#pragma unroll
        for (int v = 0; v < S::kVec; ++v) {
            if (head_of[v] < heads_valid) {
                m_loc[v] = fmaxf(m_loc[v], ml[head_of[v] * 2]);
            }
        }
    }
    for (int i = warp; i < n; i += S::kWarps) {
        const float *rec = base + static_cast<long long>(i) * S::kRec;
#pragma unroll
        for (int v = 0; v < S::kVec; ++v) {
            if (head_of[v] < heads_valid) {
                const float2 ml = *reinterpret_cast<const float2 *>(rec + S::kMl + head_of[v] * 2);
                const float w = exp2f(ml.x - m_loc[v]);
                const float4 x = *reinterpret_cast<const float4 *>(rec + head_of[v] * VD + slice0 + ((v * 32 + lane) % (HD / 4)) * 4);
                acc[v].x = fmaf(w, x.x, acc[v].x);
                acc[v].y = fmaf(w, x.y, acc[v].y);
                acc[v].z = fmaf(w, x.z, acc[v].z);
                acc[v].w = fmaf(w, x.w, acc[v].w);
                l_loc[v] = fmaf(w, ml.y, l_loc[v]);
            }
        }
    }
#pragma unroll
    for (int v = 0; v < S::kVec; ++v) {
        acc_s[warp][v * 32 + lane] = acc[v];
        if ((v * 32 + lane) % (HD / 4) == 0) {
            m_s[warp][head_of[v]] = m_loc[v];
            l_s[warp][head_of[v]] = l_loc[v];
        }
    }
    __syncthreads();

    for (int f = threadIdx.x; f < S::kFloats / 4; f += S::kWarps * 32) {
        const int head = f / (HD / 4);
        if (head >= heads_valid) {
            continue;
        }
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < S::kWarps; ++w) {
            m_all = fmaxf(m_all, m_s[w][head]);
        }
        float4 o4 = make_float4(0.f, 0.f, 0.f, 0.f);
        float l_all = 0.f;
#pragma unroll
        for (int w = 0; w < S::kWarps; ++w) {
            const float mw = m_s[w][head];
            if (mw != -INFINITY) {
                const float wgt = exp2f(mw - m_all);
                const float4 x = acc_s[w][f];
                o4.x = fmaf(wgt, x.x, o4.x);
                o4.y = fmaf(wgt, x.y, o4.y);
                o4.z = fmaf(wgt, x.z, o4.z);
                o4.w = fmaf(wgt, x.w, o4.w);
                l_all = fmaf(wgt, l_s[w][head], l_all);
            }
        }
        const float inv = 1.f / l_all;
        const int q_head = kv_head * p.group_size + head_tile * HPT + head;
        const long long off = s * p.o_seq_stride + q_head * p.o_head_stride + slice0 + (f % (HD / 4)) * 4;
        const uint32_t lo = packPair(o4.x * inv, o4.y * inv, T());
        const uint32_t hi = packPair(o4.z * inv, o4.w * inv, T());
        for (int d = 0; d <= p.num_extra_out; ++d) { // the output and every further destination
            T *out = static_cast<T *>(d == 0 ? p.out : p.extra_out[d - 1]) + off;
            *reinterpret_cast<uint32_t *>(out) = lo;
            *reinterpret_cast<uint32_t *>(out + 2) = hi;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
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

// 4-D map {head_size, block_size, num_kv_heads, num_blocks} over one cache pool, or (row_boxes) the 5-D map
// {64, block_size, width / 64, num_kv_heads, num_blocks} whose box is every column chunk of 16 rows.
bool encodeCacheMap(CUtensorMap *map, const Info &I, const void *base,
                    ptrdiff_t row_stride, ptrdiff_t head_stride, ptrdiff_t block_stride, size_t width, bool row_boxes) {
    EncodeTiledFn fn = encodeTiled();
    if (fn == nullptr) {
        return false;
    }
    if (row_boxes) {
        const cuuint64_t dims[5] = {64, I.block_size, width / 64, I.num_kv_heads, I.num_blocks};
        const cuuint64_t strides[4] = {static_cast<cuuint64_t>(row_stride) * 2, 128, static_cast<cuuint64_t>(head_stride) * 2,
                                       static_cast<cuuint64_t>(block_stride) * 2};
        const cuuint32_t box[5] = {64, kTileTokens, static_cast<cuuint32_t>(width / 64), 1, 1};
        const cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
        const CUtensorMapDataType dt = (I.dtype == INFINI_DTYPE_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        return fn(map, dt, 5, const_cast<void *>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    const cuuint64_t dims[4] = {width, I.block_size, I.num_kv_heads, I.num_blocks};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(row_stride) * 2, static_cast<cuuint64_t>(head_stride) * 2,
                                   static_cast<cuuint64_t>(block_stride) * 2};
    const cuuint32_t box[4] = {64, kTileTokens, 1, 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = (I.dtype == INFINI_DTYPE_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const CUresult rc = fn(map, dt, 4, const_cast<void *>(base), dims, strides, box, elem_strides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

int envInt(const char *name, int fallback, int lo, int hi) {
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') {
        return fallback;
    }
    const long parsed = std::strtol(v, nullptr, 10);
    if (parsed < lo || parsed > hi) {
        return fallback;
    }
    return static_cast<int>(parsed);
}

size_t roundUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct WorkspaceLayout {
    size_t header_off, prefix_off, range_off, task_off, counter_off, partial_off, total;
};

WorkspaceLayout workspaceLayout(const Info &I, const StreamPlan &plan) {
    WorkspaceLayout L;
    const size_t units = I.num_seqs * I.num_kv_heads * static_cast<size_t>(plan.head_tiles_per_group);
    L.header_off = 0;
    L.prefix_off = 256;
    L.range_off = roundUp(L.prefix_off + (I.num_seqs + 1) * sizeof(long long), 256);
    L.task_off = roundUp(L.range_off + static_cast<size_t>(plan.num_workers) * sizeof(int4), 256);
    L.counter_off = roundUp(L.task_off + static_cast<size_t>(plan.num_workers) * sizeof(int4), 256);
    // the wide-head kernel has no counters
    L.partial_off = roundUp(L.counter_off + (plan.wide ? 0 : (units + 1) * sizeof(int)), 256);
    const size_t rec = static_cast<size_t>(plan.heads_per_tile) * (I.value_size + 2) * sizeof(float);
    const size_t pieces = static_cast<size_t>(plan.num_workers) * (plan.max_chunks + 1);
    L.total = roundUp(L.partial_off + (units + pieces) * rec, 256);
    return L;
}

template <typename T, int HD, int HPT>
infiniStatus_t launchTyped(const StreamPlan &plan, const StreamArgs &args, const CUtensorMap &mk, const CUtensorMap &mv,
                           int device_id, cudaStream_t stream) {
    // The opt-in shared memory limit is a per-device, per-kernel attribute; raise it whenever a plan
    // needs more than any earlier plan on that device did.
    static std::mutex attr_mutex;
    static size_t attr_bytes[2][64] = {};
    const int pool = args.max_chunks > 0 ? 1 : 0;
    auto kernel = pool ? pagedDecodeStreamKernel<T, HD, HPT, true> : pagedDecodeStreamKernel<T, HD, HPT, false>;
    {
        std::lock_guard<std::mutex> lock(attr_mutex);
        const bool tracked = device_id >= 0 && device_id < 64;
        if (!tracked || attr_bytes[pool][device_id] < plan.smem_bytes) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes)) != cudaSuccess) {
                return checkLaunch("cudaFuncSetAttribute(pagedDecodeStreamKernel)");
            }
            if (tracked) {
                attr_bytes[pool][device_id] = plan.smem_bytes;
            }
        }
    }
    // All launches carry the programmatic-serialization attribute: each kernel's prologue overlaps
    // the tail of whatever precedes it in the stream, and each kernel waits (griddepcontrol.wait)
    // before it reads anything a predecessor may have written.
    cudaLaunchAttribute pdl;
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl.val.programmaticStreamSerializationAllowed = plan.use_pdl ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = stream;
    cfg.attrs = &pdl;
    cfg.numAttrs = 1;

    // reset kernel: the chunk counter, the per-unit tile counters when units are merged inside the main
    // kernel, the error flag
    const long long units = static_cast<long long>(args.p.num_seqs) * args.units_per_seq;
    // (nothing to clear when the units are merged by the combine kernel and ranges are not cut into pieces:
    // small and long-context calls are launch-bound, and a kernel that does nothing still costs microseconds)
    if (args.merge_in_kernel || pool) {
        const long long count = 1 + (args.merge_in_kernel ? units : 0);
        long long ctas = (count + 4 * kResetThreads - 1) / (4 * kResetThreads);
        cfg.gridDim = dim3(static_cast<unsigned>(ctas > 64 ? 64 : ctas));
        cfg.blockDim = dim3(kResetThreads);
        cfg.dynamicSmemBytes = 0;
        if (cudaLaunchKernelEx(&cfg, pagedDecodeResetKernel, args, count) != cudaSuccess) {
            return checkLaunch("pagedDecodeResetKernel");
        }
    }
    if (!plan.embedded_plan) {
        cfg.gridDim = dim3(1);
        cfg.blockDim = dim3(kPlanThreads);
        cfg.dynamicSmemBytes = 0;
        if (cudaLaunchKernelEx(&cfg, pagedDecodePlanKernel, args) != cudaSuccess) {
            return checkLaunch("pagedDecodePlanKernel");
        }
    }
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(plan.warps_per_cta * 32);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    if (cudaLaunchKernelEx(&cfg, kernel, mk, mv, args) != cudaSuccess) {
        return checkLaunch("pagedDecodeStreamKernel");
    }
    if (args.merge_in_kernel) {
        return checkLaunch("pagedDecodeStream");
    }
    // One CTA per unit merges the unit's records (a unit that one piece covered has none and its CTA
    // leaves at once).  Few units cut into many pieces each (a handful of very long sequences): several
    // CTAs per unit, 32 value columns each.  Records of 16 heads are always merged in slices (a whole
    // record does not fit one CTA's shared memory).
    cfg.dynamicSmemBytes = 0;
    constexpr int kWideSlice = (HD >= 64) ? 64 : HD;
    if (units * 4 <= plan.num_workers) {
        cfg.gridDim = dim3(static_cast<unsigned>(units), HD / 32);
        cfg.blockDim = dim3(CombineShape<32, HD, HPT>::kWarps * 32);
        if (cudaLaunchKernelEx(&cfg, pagedDecodeCombineKernel<T, 32, HD, HPT, true>, args) != cudaSuccess) {
            return checkLaunch("pagedDecodeCombineKernel");
        }
    } else if (HPT == 16) {
        cfg.gridDim = dim3(static_cast<unsigned>(units), HD / kWideSlice);
        cfg.blockDim = dim3(CombineShape<kWideSlice, HD, HPT>::kWarps * 32);
        if (cudaLaunchKernelEx(&cfg, pagedDecodeCombineKernel<T, kWideSlice, HD, HPT, true>, args) != cudaSuccess) {
            return checkLaunch("pagedDecodeCombineKernel");
        }
    } else {
        cfg.gridDim = dim3(static_cast<unsigned>(units));
        cfg.blockDim = dim3(CombineShape<HD, HD, 8>::kWarps * 32);
        if (cudaLaunchKernelEx(&cfg, pagedDecodeCombineKernel<T, HD, HD, 8, true>, args) != cudaSuccess) {
            return checkLaunch("pagedDecodeCombineKernel");
        }
    }
    return checkLaunch("pagedDecodeStream");
}

template <typename T, int KD, int VD>
infiniStatus_t launchWide(const StreamPlan &plan, const StreamArgs &args, const CUtensorMap &mk, const CUtensorMap &mv,
                          int device_id, cudaStream_t stream) {
    static std::mutex attr_mutex;
    static size_t attr_bytes[64] = {};
    auto kernel = pagedDecodeWideKernel<T, KD, VD>;
    {
        std::lock_guard<std::mutex> lock(attr_mutex);
        const bool tracked = device_id >= 0 && device_id < 64;
        if (!tracked || attr_bytes[device_id] < plan.smem_bytes) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes)) != cudaSuccess) {
                return checkLaunch("cudaFuncSetAttribute(pagedDecodeWideKernel)");
            }
            if (tracked) {
                attr_bytes[device_id] = plan.smem_bytes;
            }
        }
    }
    cudaLaunchAttribute pdl;
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl.val.programmaticStreamSerializationAllowed = plan.use_pdl ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = stream;
    cfg.attrs = &pdl;
    cfg.numAttrs = 1;
    // the plan always comes from the one-CTA plan kernel here
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(kPlanThreads);
    cfg.dynamicSmemBytes = 0;
    if (cudaLaunchKernelEx(&cfg, pagedDecodePlanKernel, args) != cudaSuccess) {
        return checkLaunch("pagedDecodePlanKernel");
    }
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(kWideWarps * 32);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    if (cudaLaunchKernelEx(&cfg, kernel, mk, mv, args) != cudaSuccess) {
        return checkLaunch("pagedDecodeWideKernel");
    }
    cfg.gridDim = dim3(plan.num_workers, VD / 64);
    cfg.blockDim = dim3(CombineShape<64, VD, kWideHeads>::kWarps * 32);
    cfg.dynamicSmemBytes = 0;
    if (cudaLaunchKernelEx(&cfg, pagedDecodeCombineKernel<T, 64, VD, kWideHeads>, args) != cudaSuccess) {
        return checkLaunch("pagedDecodeCombineKernel");
    }
    return checkLaunch("pagedDecodeWide");
}

} // namespace

StreamPlan planStream(const Info &I, const DeviceProps &props) {
    StreamPlan plan;
    const size_t hd = I.head_size;
    const bool wide = (hd == 576 && (I.value_size == 576 || I.value_size == 512));
    if (!wide && (I.value_size != hd || (hd != 64 && hd != 128 && hd != 192 && hd != 256))) {
        return plan;
    }
    if (I.block_size % kTileTokens != 0 || I.num_seqs == 0 || I.num_heads == 0) {
        return plan;
    }
    auto even = [](ptrdiff_t v) { return (v & 1) == 0; };
    auto mult8 = [](ptrdiff_t v) { return v > 0 && (v % 8) == 0; }; // 16 bytes of a 2-byte dtype
    if (!even(I.q_seq_stride) || !even(I.q_head_stride) || !even(I.o_seq_stride) || !even(I.o_head_stride)) {
        return plan;
    }
    if (!mult8(I.k_row_stride) || !mult8(I.k_head_stride) || !mult8(I.k_block_stride)
        || !mult8(I.v_row_stride) || !mult8(I.v_head_stride) || !mult8(I.v_block_stride)) {
        return plan;
    }
    if (I.num_blocks == 0) {
        return plan;
    }
    // Total tiles must stay far from 64-bit overflow and per-sequence tiles must fit an int.
    const unsigned long long tiles_per_seq_max = static_cast<unsigned long long>(I.max_num_blocks_per_seq) * (I.block_size / kTileTokens);
    if (tiles_per_seq_max > 0x3fffffffull) {
        return plan;
    }
    // Trial encode with a stand-in base address: checks that the driver accepts these strides.
    CUtensorMap probe;
    void *fake = reinterpret_cast<void *>(static_cast<uintptr_t>(1) << 30);
    if (!encodeCacheMap(&probe, I, fake, I.k_row_stride, I.k_head_stride, I.k_block_stride, hd, false)
        || !encodeCacheMap(&probe, I, fake, I.v_row_stride, I.v_head_stride, I.v_block_stride, I.value_size, false)) {
        return plan;
    }
    // One copy per tensor and tile (the 5-D maps, where the driver takes them) for key width 576, whose tile is
    // 9 + 8 chunks: 13 % faster at 128 heads x 64 x 4096 tokens, 8 % at 16 heads.  At head 64 / 128 (1 or 2 chunks
    // per tensor) it measured the same to 1.4 % slower, so those keep one copy per chunk.
    // INFINIOP_PAGED_DECODE_ROW_BOXES = 0 | 1 overrides either way.
    plan.row_boxes = envInt("INFINIOP_PAGED_DECODE_ROW_BOXES", wide ? 1 : 0, 0, 1) != 0
                     && encodeCacheMap(&probe, I, fake, I.k_row_stride, I.k_head_stride, I.k_block_stride, hd, true)
                     && encodeCacheMap(&probe, I, fake, I.v_row_stride, I.v_head_stride, I.v_block_stride, I.value_size, true);
    if (wide && (!mult8(I.q_seq_stride) || !mult8(I.q_head_stride))) {
        return plan; // q rows are copied 16 bytes at a time
    }
    if (wide) {
        // one worker = one CTA of four warps sharing a ring of 36 KiB (34 KiB) tiles
        const int group = static_cast<int>(I.num_heads / I.num_kv_heads);
        plan.wide = true;
        plan.heads_per_tile = kWideHeads;
        plan.head_tiles_per_group = (group + kWideHeads - 1) / kWideHeads;
        plan.warps_per_cta = kWideWarps;
        plan.stages = envInt("INFINIOP_PAGED_DECODE_STAGES", kWideDefaultStages, 2, 4);
        plan.embedded_plan = false;
        plan.use_pdl = envInt("INFINIOP_PAGED_DECODE_PDL", 1, 0, 1) != 0;
        const size_t stage_bytes = (hd / 64 + I.value_size / 64) * kTileTokens * 128;
        // the unit's Q rows, padded, and the two buffers of four 1 KiB partial score tiles
        const size_t q_bytes = kWideHeads * (hd * 2 + 16) + 2 * kWideWarps * kWideHeads * kTileTokens * 4;
        auto smemFor = [&](int stages) { return static_cast<size_t>(stages) * (stage_bytes + 16) + q_bytes + 1024; };
        while (plan.stages > 2 && smemFor(plan.stages) > props.smem_per_block_optin) {
            --plan.stages;
        }
        if (smemFor(plan.stages) > props.smem_per_block_optin) {
            plan.wide = false;
            return plan;
        }
        // the wanted number of resident CTAs comes first: the ring gives up slots (down to 2) to fit them
        int ctas_per_sm = envInt("INFINIOP_PAGED_DECODE_CTAS_PER_SM", 2, 1, 4);
        while (plan.stages > 2 && ctas_per_sm * (smemFor(plan.stages) + 1024) > props.smem_per_sm) {
            --plan.stages;
        }
        plan.smem_bytes = smemFor(plan.stages);
        while (ctas_per_sm > 1 && ctas_per_sm * (plan.smem_bytes + 1024) > props.smem_per_sm) {
            --ctas_per_sm;
        }
        plan.grid = props.sm_count * ctas_per_sm;
        plan.num_workers = plan.grid;
        plan.workspace_bytes = workspaceLayout(I, plan).total;
        plan.eligible = true;
        return plan;
    }

    const int group = static_cast<int>(I.num_heads / I.num_kv_heads);
    // Groups of more than 8 q-heads per kv-head use all 16 rows of the MMA (head sizes up to 128, where
    // the second row's Q fragments still fit the registers): K/V are re-read once per 16 heads, not per 8.
    plan.heads_per_tile = (group > kHeadsPerTile && hd <= 128 && envInt("INFINIOP_PAGED_DECODE_HEADS_PER_TILE", 16, 8, 16) == 16) ? 16 : kHeadsPerTile;
    plan.head_tiles_per_group = (group + plan.heads_per_tile - 1) / plan.heads_per_tile;

    const size_t stage_bytes = 2 * (hd / 64) * kTileTokens * 128;
    const int default_stages = 2;
    plan.warps_per_cta = envInt("INFINIOP_PAGED_DECODE_WARPS", 4, 1, hd == 64 ? 4 : kMaxWarps);
    plan.stages = envInt("INFINIOP_PAGED_DECODE_STAGES", default_stages, 1, kMaxStages);
    // Head 64 halves the bytes per tile while the per-tile latencies stay: a third resident CTA per SM
    // (its registers allow it) keeps enough copies in flight - 5.5 TB/s instead of 4.2 at 64 x 4096 tokens.
    int ctas_per_sm = envInt("INFINIOP_PAGED_DECODE_CTAS_PER_SM", hd == 64 ? 3 : 2, 1, 8);
    // The plan is derived inside the main kernel (one launch fewer) when the per-sequence prefix fits
    // a modest slice of shared memory; larger batches use the separate one-CTA plan kernel.
    plan.embedded_plan = envInt("INFINIOP_PAGED_DECODE_EMBEDDED_PLAN", 1, 0, 1) != 0 && I.num_seqs <= 4095;
    plan.use_pdl = envInt("INFINIOP_PAGED_DECODE_PDL", 1, 0, 1) != 0;
    // Pieces (off by default: INFINIOP_PAGED_DECODE_CHUNKS = 1..8 turns them on): the last eighth of every
    // range goes to the shared pool in that many chunks of halving size.  A chunk is located by a binary
    // search over the tile prefix, which only the embedded plan keeps in shared memory: with the separate
    // plan kernel ranges stay whole.  Measured: the pool evens the workers' finishing times out (they spread
    // over 5 us instead of 36 at 64 x 4096 tokens), but every piece that does not cover a whole unit leaves
    // a record, and reading ten records per unit instead of three costs what the balance gains; with more
    // units than workers it changed the step by -2 % to +4 % from one GPU of the pool to the next.
    plan.max_chunks = plan.embedded_plan ? envInt("INFINIOP_PAGED_DECODE_CHUNKS", 0, 0, 8) : 0;
    plan.min_chunk = envInt("INFINIOP_PAGED_DECODE_MIN_CHUNK", 4, 1, 1024);
    plan.tail_shift = envInt("INFINIOP_PAGED_DECODE_TAIL_SHIFT", 3, 1, 6);
    plan.merge_in_kernel = envInt("INFINIOP_PAGED_DECODE_MERGE_IN_KERNEL", 1, 0, 1) != 0;
    plan.l2_evict_first = envInt("INFINIOP_PAGED_DECODE_L2_EVICT_FIRST", 1, 0, 1) != 0;
    // How long a worker waits for one of its own copies before it gives up (INFINIOP_PAGED_DECODE_WAIT_LIMIT_MS,
    // default 2000), counted on the SM's cycle counter at a nominal 2 GHz.  And a switch for the test of that
    // path only: INFINIOP_PAGED_DECODE_TEST_WITHHOLD_COPY=1 makes worker 0 leave out the first copy it would
    // issue, so that its first wait runs out, the kernel returns and the device's status word says so.
    plan.wait_limit_cycles = static_cast<long long>(envInt("INFINIOP_PAGED_DECODE_WAIT_LIMIT_MS", 2000, 1, 60000)) * 2000000ll;
    plan.withhold_first_copy = envInt("INFINIOP_PAGED_DECODE_TEST_WITHHOLD_COPY", 0, 0, 1) != 0;
    const size_t plan_bytes = plan.embedded_plan ? (I.num_seqs + 1 + kMaxWarps) * sizeof(long long) : 0;
    auto smemFor = [&](int warps, int stages) { return static_cast<size_t>(warps) * (stages * (stage_bytes + 8) + kMergeList * sizeof(long long)) + plan_bytes + 1024; };
    const size_t budget = props.smem_per_block_optin;
    while (plan.stages > 1 && smemFor(plan.warps_per_cta, plan.stages) > budget) {
        --plan.stages;
    }
    if (smemFor(plan.warps_per_cta, plan.stages) > budget) {
        return plan;
    }
    plan.smem_bytes = smemFor(plan.warps_per_cta, plan.stages);
    // Each resident CTA also reserves 1 KiB of system shared memory.
    while (ctas_per_sm > 1 && ctas_per_sm * (plan.smem_bytes + 1024) > props.smem_per_sm) {
        --ctas_per_sm;
    }
    plan.grid = props.sm_count * ctas_per_sm;
    plan.num_workers = plan.grid * plan.warps_per_cta;
    // a worker counts the tiles of its range in 32 bits
    const unsigned long long units_per_seq = static_cast<unsigned long long>(I.num_kv_heads) * plan.head_tiles_per_group;
    if (static_cast<unsigned long long>(I.num_seqs) * tiles_per_seq_max * units_per_seq / plan.num_workers >= 0x7fffffffull) {
        return plan;
    }
    plan.workspace_bytes = workspaceLayout(I, plan).total;
    plan.eligible = true;
    return plan;
}

bool streamTakesPointers(const StreamPlan &plan, const DecodeParams &p, const void *workspace) {
    const auto addr = [](const void *ptr) { return reinterpret_cast<uintptr_t>(ptr); };
    // TMA needs 16-byte aligned pool bases; the fragment loads need 4-byte aligned q/out (the wide-head
    // kernel copies q rows 16 bytes at a time).
    const uintptr_t q_mask = plan.wide ? 15u : 3u;
    uintptr_t outs = addr(p.out);
    for (int d = 0; d < p.num_extra_out; ++d) {
        outs |= addr(p.extra_out[d]);
    }
    return ((addr(p.k_cache) | addr(p.v_cache)) & 15u) == 0 && (addr(p.q) & q_mask) == 0 && (outs & 3u) == 0
           && (addr(workspace) & 255u) == 0;
}

infiniStatus_t launchDecodeStream(const Info &I, const StreamPlan &plan, const DecodeParams &p,
                                  void *workspace, size_t workspace_size, cudaStream_t stream) {
    B200_RETURN_IF(workspace_size < plan.workspace_bytes, INFINI_STATUS_INSUFFICIENT_WORKSPACE);
    if (!streamTakesPointers(plan, p, workspace)) {
        B200_RETURN_IF(p.new_k != nullptr, INFINI_STATUS_INTERNAL_ERROR); // the append form checks before it gets here
        return launchDecodeGeneric(I, p, stream);
    }
    CUtensorMap mk, mv;
    B200_RETURN_IF(!encodeCacheMap(&mk, I, p.k_cache, I.k_row_stride, I.k_head_stride, I.k_block_stride, I.head_size, plan.row_boxes), INFINI_STATUS_INTERNAL_ERROR);
    B200_RETURN_IF(!encodeCacheMap(&mv, I, p.v_cache, I.v_row_stride, I.v_head_stride, I.v_block_stride, I.value_size, plan.row_boxes), INFINI_STATUS_INTERNAL_ERROR);

    const WorkspaceLayout L = workspaceLayout(I, plan);
    auto *ws = static_cast<unsigned char *>(workspace);
    StreamArgs a;
    a.p = p;
    a.header = reinterpret_cast<PlanHeader *>(ws + L.header_off);
    a.prefix = reinterpret_cast<long long *>(ws + L.prefix_off);
    a.range_start = reinterpret_cast<int4 *>(ws + L.range_off);
    a.tasks = reinterpret_cast<int4 *>(ws + L.task_off);
    a.counters = reinterpret_cast<int *>(ws + L.counter_off);
    a.partials = reinterpret_cast<float *>(ws + L.partial_off);
    a.head_tiles = plan.head_tiles_per_group;
    a.units_per_seq = static_cast<int>(I.num_kv_heads) * plan.head_tiles_per_group;
    a.tiles_per_page = static_cast<int>(I.block_size / kTileTokens);
    a.stages = plan.stages;
    a.row_boxes = plan.row_boxes ? 1 : 0;
    a.num_workers = plan.num_workers;
    a.embedded_plan = plan.embedded_plan ? 1 : 0;
    a.max_chunks = plan.max_chunks;
    a.min_chunk = plan.min_chunk;
    a.tail_shift = plan.tail_shift;
    a.l2_evict_first = plan.l2_evict_first ? 1 : 0;
    a.wait_limit_cycles = plan.wait_limit_cycles;
    a.withhold_first_copy = plan.withhold_first_copy ? 1 : 0;
    // Units cut into a few pieces each are merged by the last worker to arrive; a handful of units cut
    // into hundreds of pieces each (4 or more workers per unit) by the combine kernel, many CTAs per unit.
    a.merge_in_kernel = (!plan.wide && plan.merge_in_kernel && static_cast<long long>(I.num_seqs) * a.units_per_seq * 4 > plan.num_workers) ? 1 : 0;

    int device_id = -1;
    (void)cudaGetDevice(&device_id);
    const bool f16 = (I.dtype == INFINI_DTYPE_F16);
    if (plan.wide) {
        if (I.value_size == 512) {
            return f16 ? launchWide<__half, 576, 512>(plan, a, mk, mv, device_id, stream)
                       : launchWide<__nv_bfloat16, 576, 512>(plan, a, mk, mv, device_id, stream);
        }
        return f16 ? launchWide<__half, 576, 576>(plan, a, mk, mv, device_id, stream)
                   : launchWide<__nv_bfloat16, 576, 576>(plan, a, mk, mv, device_id, stream);
    }
    const bool h16 = plan.heads_per_tile == 16;
    switch (I.head_size) {
    case 64:
        if (h16) {
            return f16 ? launchTyped<__half, 64, 16>(plan, a, mk, mv, device_id, stream) : launchTyped<__nv_bfloat16, 64, 16>(plan, a, mk, mv, device_id, stream);
        }
        return f16 ? launchTyped<__half, 64, 8>(plan, a, mk, mv, device_id, stream) : launchTyped<__nv_bfloat16, 64, 8>(plan, a, mk, mv, device_id, stream);
    case 128:
        if (h16) {
            return f16 ? launchTyped<__half, 128, 16>(plan, a, mk, mv, device_id, stream) : launchTyped<__nv_bfloat16, 128, 16>(plan, a, mk, mv, device_id, stream);
        }
        return f16 ? launchTyped<__half, 128, 8>(plan, a, mk, mv, device_id, stream) : launchTyped<__nv_bfloat16, 128, 8>(plan, a, mk, mv, device_id, stream);
    case 192:
        return f16 ? launchTyped<__half, 192, 8>(plan, a, mk, mv, device_id, stream) : launchTyped<__nv_bfloat16, 192, 8>(plan, a, mk, mv, device_id, stream);
    case 256:
        return f16 ? launchTyped<__half, 256, 8>(plan, a, mk, mv, device_id, stream) : launchTyped<__nv_bfloat16, 256, 8>(plan, a, mk, mv, device_id, stream);
    default:
        return INFINI_STATUS_BAD_TENSOR_SHAPE;
    }
}

} // namespace b200::paged_attention
