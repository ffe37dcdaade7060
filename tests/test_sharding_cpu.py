"""Host-side logic of the multi-GPU (sequence-sharded) path, run as two gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from infinicore_b200 import sharding, workloads


def test_round_robin_and_balanced_partition_every_sequence_once():
    lens = workloads.config5_lengths(num_seqs=257).tolist()
    for policy in ("round_robin", "balanced"):
        for world in (1, 2, 4, 8):
            shards = [sharding.shard(lens, r, world, policy) for r in range(world)]
            flat = sorted(i for s in shards for i in s)
            assert flat == list(range(257))
    rr = sharding.round_robin(10, 4)
    assert rr == [[0, 4, 8], [1, 5, 9], [2, 6], [3, 7]]


def test_balanced_policy_equalises_tokens_on_ragged_lengths():
    lens = [32768, 16, 16, 16, 20000, 9000, 3000, 700, 100, 16]
    world = 2
    per_rank = lambda shards: [sum(lens[i] for i in s) for s in shards]
    rr = per_rank(sharding.round_robin(len(lens), world))
    bal = per_rank(sharding.balanced_by_tokens(lens, world))
    assert max(bal) <= max(rr)
    assert max(bal) - min(bal) <= max(lens)


def test_config5_shards_are_consistent_across_ranks():
    world = 4
    all_lens = workloads.config5_lengths(num_seqs=64)
    total = 0
    for rank in range(world):
        c = workloads.config5_shard(rank, world, device="cpu", num_seqs=64)
        assert torch.equal(c.seq_lens, all_lens[rank::world])
        total += c.total_tokens
        # every rank owns its own pool: block ids are local and distinct within the rank
        used = torch.cat([c.block_tables[i, : (int(n) + 15) // 16] for i, n in enumerate(c.seq_lens)])
        assert used.unique().numel() == used.numel() and int(used.max()) < c.k_cache.shape[0]
    assert total == int(all_lens.sum())


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens = workloads.config5_lengths(num_seqs=96).tolist()
        mine = sharding.shard(lens, rank, world)
        my_bytes = float(sharding.kv_bytes([lens[i] for i in mine], 8, 128, 128, 2))
        my_ms = 1.0 + rank  # pretend rank 1 is the slow one
        # what bench.py does: SUM of bytes, MAX of time, over ranks
        b = torch.tensor([my_bytes], dtype=torch.float64)
        t = torch.tensor([my_ms], dtype=torch.float64)
        dist.all_reduce(b, op=dist.ReduceOp.SUM)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        if rank == 0:
            out.put((float(b), float(t), gathered))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_aggregate_like_the_bench():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    total_bytes, slowest_ms, gathered = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    lens = workloads.config5_lengths(num_seqs=96).tolist()
    assert sorted(gathered[0] + gathered[1]) == list(range(96))
    assert total_bytes == sharding.kv_bytes(lens, 8, 128, 128, 2)
    assert slowest_ms == 2.0
    per_rank_bytes = [sharding.kv_bytes([lens[i] for i in g], 8, 128, 128, 2) for g in gathered]
    assert sharding.job_throughput(per_rank_bytes, [1.0, 2.0]) == pytest.approx(total_bytes / 2e-3 / 1e9)


def test_a_rank_that_dies_before_the_step_is_reported_by_the_parent():
    """Failure detection on the host: a worker that exits before joining is seen as a non-zero exit
    code by the launcher; nothing is left waiting on a device."""
    ctx = mp.get_context("spawn")
    p = ctx.Process(target=_dies)
    p.start()
    p.join(timeout=60)
    assert p.exitcode == 3


def _dies():
    raise SystemExit(3)


# ---- optional KV-head-sharded mode: slices + all-gather reproduce the unsharded result ----------

def _head_worker(rank, world, port, out):
    import numpy as np

    import oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = workloads.build_case("hs", dtype=torch.float16, seq_lens=[40, 7, 129], num_heads=8, num_kv_heads=4,
                                 head_size=64, block_size=16, seed=81)  # same seed: every rank sees the same full problem

        def bits(t):
            return t.contiguous().view(torch.int16).numpy().view(np.uint16)

        qs, ks = sharding.head_slices(8, 4, rank, world)
        local = oracle.paged_attention(bits(c.q[:, qs]), bits(c.k_cache[:, ks]), bits(c.v_cache[:, ks]),
                                       c.block_tables.numpy(), c.seq_lens.numpy(), c.scale, 12)
        full = sharding.gather_head_sharded(torch.from_numpy(local), world)
        if rank == 0:
            want = oracle.paged_attention(bits(c.q), bits(c.k_cache), bits(c.v_cache), c.block_tables.numpy(),
                                          c.seq_lens.numpy(), c.scale, 12)
            out.put(bool(np.array_equal(full.numpy(), want)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_head_sharded_outputs_all_gather_to_the_unsharded_result():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_head_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    assert out.get(timeout=180) is True
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0


def test_head_slices():
    assert sharding.head_slices(64, 8, 3, 8) == (slice(24, 32), slice(3, 4))
    assert sharding.head_slices(32, 8, 1, 2) == (slice(16, 32), slice(4, 8))
    with pytest.raises(ValueError):
        sharding.head_slices(32, 8, 0, 3)
