"""libinfiniccl.so (InfiniCCL C ABI over NCCL) on real devices, in the manner of the reference's
src/infiniccl-test: one host thread per device, every collective checked against the values the
ranks put in.  Runs on every visible GPU up to 4: with one GPU the group has one rank (each
collective is then a copy), with two or more the data really crosses NVLink."""
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _world():
    return max(1, min(torch.cuda.device_count(), 4))


@pytest.fixture(scope="module")
def comms():
    from infinicore_b200 import ccl

    group = ccl.init_all(list(range(_world())))
    yield group
    for c in group:
        torch.cuda.synchronize(c.device)
        c.destroy()


def _run_ranks(comms, fn):
    """fn(comm) on one thread per rank; collects results, re-raises the first failure."""
    results, errors = [None] * len(comms), []

    def body(c):
        try:
            torch.cuda.set_device(c.device)
            results[c.rank] = fn(c)
            torch.cuda.synchronize(c.device)
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=body, args=(c,)) for c in comms]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads), "a rank did not finish"
    if errors:
        raise errors[0]
    return results


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int32, torch.int64])
def test_all_reduce_sum_and_max(comms, dtype):
    from infinicore_b200 import ccl

    n, world = 4099, len(comms)

    def fn(c):
        x = (torch.arange(n, device=f"cuda:{c.device}") % 7 + c.rank).to(dtype)
        s, m = torch.empty_like(x), torch.empty_like(x)
        c.all_reduce(x, s, ccl.SUM)
        c.all_reduce(x, m, ccl.MAX)
        return s.cpu(), m.cpu()

    base = (torch.arange(n) % 7)
    want_sum = sum((base + r).to(dtype) for r in range(world))
    want_max = (base + world - 1).to(dtype)
    for s, m in _run_ranks(comms, fn):
        assert torch.equal(s, want_sum)
        assert torch.equal(m, want_max)


def test_all_gather_is_rank_major_and_restores_head_order(comms):
    """The head-sharded decode mode: per-rank [seqs, heads / N, d] -> [seqs, heads, d]."""
    from infinicore_b200 import sharding

    world, seqs, hpr, d = len(comms), 5, 3, 128

    def fn(c):
        dev = f"cuda:{c.device}"
        full = torch.arange(seqs * world * hpr * d, dtype=torch.float32, device=dev).reshape(seqs, world * hpr, d).to(torch.bfloat16)
        local = full[:, c.rank * hpr:(c.rank + 1) * hpr].contiguous()
        got = sharding.gather_head_sharded(local, world, comm=c)
        return torch.equal(got, full)

    assert all(_run_ranks(comms, fn))


def test_broadcast_and_variable_count_collectives(comms):
    from infinicore_b200 import ccl

    world = len(comms)
    counts = [3 + 2 * r for r in range(world)]

    def fn(c):
        dev = f"cuda:{c.device}"
        # broadcast from the last rank
        src = torch.full((17,), float(c.rank), device=dev)
        dst = torch.empty_like(src)
        c.broadcast(src, dst, root=world - 1)
        # all-gather-v: rank r contributes counts[r] copies of r
        mine = torch.full((counts[c.rank],), c.rank, dtype=torch.int32, device=dev)
        gathered = torch.empty((sum(counts),), dtype=torch.int32, device=dev)
        c.all_gather_v(mine, gathered, counts)
        # reduce-scatter (equal and variable): every rank sends arange, rank r keeps slice r summed over ranks
        send = torch.arange(world * 4, dtype=torch.float32, device=dev)
        rs = torch.empty((4,), dtype=torch.float32, device=dev)
        c.reduce_scatter(send, rs, ccl.SUM)
        send_v = torch.arange(sum(counts), dtype=torch.float32, device=dev)
        rs_v = torch.empty((counts[c.rank],), dtype=torch.float32, device=dev)
        c.reduce_scatter_v(send_v, rs_v, counts, ccl.SUM)
        return dst.cpu(), gathered.cpu(), rs.cpu(), rs_v.cpu()

    want_gather = torch.cat([torch.full((counts[r],), r, dtype=torch.int32) for r in range(world)])
    offs = np.concatenate([[0], np.cumsum(counts)])
    for r, (dst, gathered, rs, rs_v) in enumerate(_run_ranks(comms, fn)):
        assert torch.equal(dst, torch.full((17,), float(world - 1)))
        assert torch.equal(gathered, want_gather)
        assert torch.equal(rs, world * torch.arange(r * 4, r * 4 + 4, dtype=torch.float32))
        assert torch.equal(rs_v, world * torch.arange(int(offs[r]), int(offs[r + 1]), dtype=torch.float32))


def test_send_recv_ring(comms):
    world = len(comms)
    if world < 2:
        pytest.skip("point-to-point needs two ranks")

    def fn(c):
        dev = f"cuda:{c.device}"
        out = torch.full((33,), float(c.rank), device=dev)
        inp = torch.empty_like(out)
        c.group_start()
        c.send(out, (c.rank + 1) % world)
        c.recv(inp, (c.rank - 1) % world)
        c.group_end()
        return inp.cpu()

    for r, inp in enumerate(_run_ranks(comms, fn)):
        assert torch.equal(inp, torch.full((33,), float((r - 1) % world)))


def test_argument_checks_return_status_codes(comms):
    from infinicore_b200 import ccl
    from infinicore_b200.libinfiniop import InfiniStatusError

    c = comms[0]
    torch.cuda.set_device(c.device)
    x = torch.zeros(8, device=f"cuda:{c.device}")
    with pytest.raises(InfiniStatusError) as e:
        c.broadcast(x, x, root=len(comms))  # root out of range
    assert e.value.status == 3  # INFINI_STATUS_BAD_PARAM
    with pytest.raises(InfiniStatusError) as e:
        ccl.check_error(ccl.lib().infinicclAllGatherV(x.data_ptr(), x.data_ptr(), (ccl.c_size_t * 1)(1), len(comms) + 1, 13,
                                                      c.handle, None))  # nranks != world size
    assert e.value.status == 3
    with pytest.raises(InfiniStatusError) as e:
        ccl.check_error(ccl.lib().infinicclAllReduce(x.data_ptr(), x.data_ptr(), 8, 1, ccl.SUM, c.handle, None))  # dtype 1 = BYTE
    assert e.value.status == 10  # INFINI_STATUS_BAD_TENSOR_DTYPE
    assert ccl.lib().infinicclCommDestroy(None) == 0  # NULL is accepted
