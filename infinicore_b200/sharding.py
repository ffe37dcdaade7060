"""Sequence sharding of a decode batch over the GPUs of one node.

The paged decode path partitions by sequence: a sequence's block table, length, q/out rows and
cache pages live on one GPU, so the ranks exchange nothing on the data path.  This module is the
host-side partitioner and the bookkeeping that turns per-rank timings into one job-level number.
(The reference has no sharding code of its own - it leaves placement to its callers; round-robin
is what benchmark configuration 5 prescribes.)
"""
from __future__ import annotations

from typing import List, Sequence


def round_robin(num_seqs: int, world: int) -> List[List[int]]:
    """Sequence i goes to rank i % world."""
    return [list(range(r, num_seqs, world)) for r in range(world)]


def balanced_by_tokens(seq_lens: Sequence[int], world: int) -> List[List[int]]:
    """Longest-first greedy: each sequence goes to the rank with the fewest tokens so far.  Equalises
    the KV bytes each GPU has to stream when lengths are ragged."""
    order = sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i))
    loads = [0] * world
    shards: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], k))
        shards[r].append(i)
        loads[r] += max(int(seq_lens[i]), 0)
    for s in shards:
        s.sort()
    return shards


def shard(seq_lens: Sequence[int], rank: int, world: int, policy: str = "round_robin") -> List[int]:
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if policy == "round_robin":
        return round_robin(len(seq_lens), world)[rank]
    if policy == "balanced":
        return balanced_by_tokens(seq_lens, world)[rank]
    raise ValueError(f"unknown sharding policy {policy!r}")


def kv_bytes(seq_lens: Sequence[int], num_kv_heads: int, head_size: int, value_size: int, elem_size: int) -> int:
    """Algorithmic bytes of one attention pass over these sequences: every K and V element once."""
    return sum(max(int(n), 0) for n in seq_lens) * num_kv_heads * (head_size + value_size) * elem_size


def job_throughput(bytes_per_rank: Sequence[float], ms_per_rank: Sequence[float]) -> float:
    """GB/s of the whole job: all ranks' bytes over the slowest rank's time."""
    return sum(bytes_per_rank) / (max(ms_per_rank) * 1e-3) / 1e9


# ---- optional KV-head-sharded mode -------------------------------------------------------------
# Rank r holds kv-heads [r * kvh / world, (r + 1) * kvh / world) of EVERY sequence and the q-heads
# that read them; its attention output is [num_seqs, num_heads / world, head_size].  The only
# exchange on the path is one all-gather of those outputs (reference collective:
# infinicclAllGather -> ncclAllGather, src/infiniccl/cuda/infiniccl_cuda.cu:219-234).

def head_slices(num_heads: int, num_kv_heads: int, rank: int, world: int):
    """(q-head slice, kv-head slice) owned by `rank`."""
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} kv-heads do not divide over {world} ranks")
    group = num_heads // num_kv_heads
    per = num_kv_heads // world
    return slice(rank * per * group, (rank + 1) * per * group), slice(rank * per, (rank + 1) * per)


def gather_head_sharded(out_local, world: int, group=None, staging=None, comm=None):
    """All-gathers per-rank outputs [num_seqs, heads_per_rank, d] into [num_seqs, heads, d].

    NCCL concatenates rank-major, so the gathered buffer is [world, num_seqs, heads_per_rank, d]; the
    head order of the full tensor is restored with a permuted view (no extra copy is made here; a
    consumer that needs contiguity pays one).  `staging` may hold a preallocated gather buffer.
    `comm` is an infinicore_b200.ccl.Communicator: the gather then goes through infinicclAllGather
    (the reference's route, src/infiniccl/cuda/infiniccl_cuda.cu:219-234) on the current stream;
    without it, through torch.distributed on `group`."""
    import torch

    num_seqs, hpr, d = out_local.shape
    if staging is None:
        staging = torch.empty((world, num_seqs, hpr, d), dtype=out_local.dtype, device=out_local.device)
    if comm is not None:
        comm.all_gather(out_local.contiguous().view(-1), staging.view(-1))
    else:
        import torch.distributed as dist

        dist.all_gather_into_tensor(staging.view(-1), out_local.contiguous().view(-1), group=group)
    return staging.permute(1, 0, 2, 3).reshape(num_seqs, world * hpr, d)


class PeerOutputs:
    """Full outputs [num_seqs, heads, d] of every rank, allocated in symmetric memory so that each
    rank can address all of them.  In the KV-head-sharded mode a rank then stores its head slice
    straight into every rank's full output from inside the attention kernels
    (infiniopPagedAttentionMultiOut) and the all-gather that would follow is replaced by one barrier.

    The exchange itself is plain stores over NVLink to peer addresses; nothing here waits on a peer
    except `barrier()`, which is torch's symmetric-memory barrier (it carries its own timeout).

    Reuse across steps.  One barrier per step orders "every rank has stored" before "this rank reads",
    but not "this rank has finished reading" before "a faster rank stores the next step's rows": with a
    single buffer a rank that is still reading step n could see rows of step n + 1.  So the outputs are
    double-buffered: `buffers` (default 2) full outputs per rank, and `advance()` moves to the next one
    after a step.  A rank can only store into buffer b again after it has passed the barrier of the step
    in between, which every rank enters only after it has issued its reads of buffer b (stream order):
    with two buffers and one barrier per step no store can overtake a read.  With `buffers=1` the caller
    must add a second cross-rank synchronisation between its reads and the next step's stores.

        peers = PeerOutputs(...)
        for step in ...:
            paged_attention_multi_out(peers.destinations(), ...)   # stores into buffer `peers.current`
            peers.barrier()
            use(peers.full)                                        # this rank's complete output of the step
            peers.advance()
    """

    def __init__(self, num_seqs: int, heads_total: int, d: int, dtype, device, group=None, buffers: int = 2):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if heads_total % self.world != 0:
            raise ValueError("heads must divide over the ranks")
        if buffers < 1:
            raise ValueError("at least one buffer")
        self.heads_per_rank = heads_total // self.world
        self.buffers = int(buffers)
        self.current = 0
        self._all = symm_mem.empty((self.buffers, num_seqs, heads_total, d), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self._all, group)
        self._slice_bytes = self.heads_per_rank * d * self._all.element_size()
        self._buffer_bytes = num_seqs * heads_total * d * self._all.element_size()

    @property
    def full(self):
        """This rank's full output in the current buffer (complete after the step's barrier)."""
        return self._all[self.current]

    def fill_(self, value):
        """Initialises every buffer of this rank (call before the first step, then synchronise all ranks)."""
        self._all.fill_(value)
        return self

    def advance(self) -> int:
        """Moves to the next buffer; call once per step, after this rank has issued its reads of `full`."""
        self.current = (self.current + 1) % self.buffers
        return self.current

    def local_slice(self):
        """This rank's heads inside its own full output (current buffer).  Every buffer's slice has the same
        shape and strides, so one attention descriptor made for it serves all of them."""
        h0 = self.rank * self.heads_per_rank
        return self.full[:, h0:h0 + self.heads_per_rank]

    def destinations(self):
        """outs for paged_attention_multi_out: the local slice first, then the address of the same
        slice inside every other rank's full output (current buffer)."""
        base = list(self.handle.buffer_ptrs)
        off = self.current * self._buffer_bytes + self.rank * self._slice_bytes
        return [self.local_slice()] + [base[r] + off for r in range(self.world) if r != self.rank]

    def barrier(self):
        """Every rank's stores have landed everywhere once all ranks have passed this point in stream order."""
        self.handle.barrier()
