// Launch interface between the paged-attention descriptor code and its CUDA kernels.
#ifndef INFINIOP_B200_PAGED_ATTENTION_KERNELS_H
#define INFINIOP_B200_PAGED_ATTENTION_KERNELS_H

#include "info.h"

#include <cuda.h>

namespace b200::paged_attention {

// Everything a decode kernel needs; strides are in ELEMENTS of the tensor's dtype.
struct DecodeParams {
    void *out;
    const void *q;
    const void *k_cache;
    const void *v_cache;
    const void *block_tables;
    const void *seq_lens;
    const float *alibi_slopes; // may be null

    int num_seqs;
    int num_heads;
    int num_kv_heads;
    int group_size; // num_heads / num_kv_heads
    int head_size;
    int value_size;
    int block_size;
    int max_blocks_per_seq;
    int index_is_64; // block_tables / seq_lens element width: 1 => 8 bytes, 0 => 4 bytes

    long long q_seq_stride, q_head_stride;
    long long o_seq_stride, o_head_stride;
    long long k_block_stride, k_head_stride, k_row_stride;
    long long v_block_stride, v_head_stride, v_row_stride;
    long long bt_seq_stride;

    float scale_log2e; // scale * log2(e): scores live in the log2 domain, softmax uses exp2

    // Decode step with append (null otherwise): row [seq, kv_head, :] of new_k / new_v is the K / V of
    // position seq_len - 1; the streaming kernel uses it instead of what the cache holds there and
    // stores it into the cache on the way.
    const void *new_k = nullptr;
    const void *new_v = nullptr;
    long long new_k_seq_stride = 0, new_v_seq_stride = 0; // head stride is head_size (dense)

    // Further destinations of every output row (same shape and strides as `out`; null otherwise).  The
    // KV-head-sharded mode stores a rank's head slice straight into every peer's full output this way,
    // so no all-gather follows the kernel.
    static constexpr int kMaxExtraOut = 7;
    void *extra_out[kMaxExtraOut] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int num_extra_out = 0;

    // Status reporting (include/infiniop/ops/kernel_status.h): the device's flag word, and whether block-table
    // entries are checked against the pool size before they are used (a bad one raises a flag and reads
    // block 0 instead).
    unsigned int *kernel_flags = nullptr;
    int check_indices = 0;
    long long num_blocks = 0;
};

// INFINIOP_PAGED_CHECK_INDICES=1 in the environment when a descriptor is created switches index checking on.
bool checkIndicesFromEnv();

// Block-table entry as the kernels use it: in checked mode an entry outside [0, num_blocks) raises
// INFINIOP_KERNEL_FLAG_BLOCK_OUT_OF_RANGE and becomes block 0.
__device__ __forceinline__ long long checkedBlock(const DecodeParams &p, long long block) {
    if (p.check_indices && static_cast<unsigned long long>(block) >= static_cast<unsigned long long>(p.num_blocks)) {
        atomicOr(p.kernel_flags, 2u);
        return 0;
    }
    return block;
}

// The same check for kernels that fetch pages through the copy engine, which fills a box outside the pool with
// zeros by itself: the entry is only reported.
__device__ __forceinline__ long long reportedBlock(const DecodeParams &p, long long block) {
    if (p.check_indices && static_cast<unsigned long long>(block) >= static_cast<unsigned long long>(p.num_blocks)) {
        atomicOr(p.kernel_flags, 2u);
    }
    return block;
}

__host__ __device__ inline long long loadIndex(const void *base, long long i, int is64) {
    return is64 ? static_cast<const long long *>(base)[i]
                : static_cast<long long>(static_cast<const int *>(base)[i]);
}

// ---- generic SIMT path (any supported head/value size, block size and strides) ---------
infiniStatus_t launchDecodeGeneric(const Info &info, const DecodeParams &p, cudaStream_t stream);

// ---- streaming path: TMA page staging + mma.sync, work split evenly over persistent warps
struct StreamPlan {
    bool eligible = false;
    int heads_per_tile = 8;       // q-heads processed together against one staged tile: 8, or 16 for groups of more than 8
    int head_tiles_per_group = 1; // ceil(group size / heads_per_tile)
    int warps_per_cta = 0;
    int stages = 0;
    int grid = 0;        // persistent CTAs
    int num_workers = 0; // grid * warps_per_cta
    size_t smem_bytes = 0;
    size_t workspace_bytes = 0;
    bool embedded_plan = false;   // the main kernel derives the plan itself (no plan kernel)
    bool use_pdl = true;          // launches carry the programmatic-serialization attribute
    bool wide = false;            // key width 576: one worker is a CTA of four warps (pagedDecodeWideKernel)
    int max_chunks = 0;           // one-warp kernel: tail chunks per range that go to the pool shared by all workers
    int min_chunk = 4;            // smallest such chunk, in 16-token tiles
    int tail_shift = 3;           // the last range_len >> tail_shift tiles of a range are cut into chunks
    bool l2_evict_first = true;   // one-warp kernel: K/V copies carry the evict-first L2 policy (they are read once)
    long long wait_limit_cycles = 4000000000ll; // a bounded mbarrier wait gives up after this many SM cycles (~2 s)
    bool withhold_first_copy = false; // test only: worker 0 never issues its first copy, so that its wait runs out
    bool row_boxes = false;   // 5-D tensor maps: one copy per tensor and tile instead of one per 64-element column chunk
    bool merge_in_kernel = true;  // split units are merged by the last worker to arrive (when few pieces per unit), not by the combine kernel
};

// Decides at descriptor creation whether the streaming path applies and sizes its workspace.
StreamPlan planStream(const Info &info, const DeviceProps &props);

infiniStatus_t launchDecodeStream(const Info &info, const StreamPlan &plan, const DecodeParams &p,
                                  void *workspace, size_t workspace_size, cudaStream_t stream);

// True when launchDecodeStream will run the streaming kernel for these pointers (and not hand the
// call to the generic kernel): the caller of the append form needs to know which one takes the rows.
bool streamTakesPointers(const StreamPlan &plan, const DecodeParams &p, const void *workspace);

// Stand-alone append for the paths that do not fuse it: position seq_len - 1 of every sequence
// receives its new_k / new_v row (one warp per row).
infiniStatus_t launchAppendNewRows(const Info &info, const DecodeParams &p, cudaStream_t stream);

} // namespace b200::paged_attention

#endif
