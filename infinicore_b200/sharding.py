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
