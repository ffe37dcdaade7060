"""The benchmark configurations at FULL size, through the C ABI, against the CPU oracle and (where the
reference's own CUDA sources were compiled into oracle/_ref) against the reference kernels run in a
child process on the same seeded inputs.

  configuration 2  bf16, 64 sequences x 4096 tokens, 32/8 heads          every row against the oracle
  configuration 3  bf16, 256 sequences, 64/8 heads, log-uniform 16..32768 every row against the oracle
  configuration 4  fp16, 2 sequences x 131072 tokens, 32/8 heads          every row; how many ways a unit was split
  configuration 5  bf16, 2048 sequences U[1024, 8192], 64/8 heads:
                   rank 0's shard of an 8-way round-robin split (256 sequences), every row;
                   the whole batch on one GPU (38.7 GB of KV, plan from the separate plan kernel), a sample of rows

Tolerance: the decode path's (fp16 atol 2e-3 / rtol 2e-3, bf16 atol 1e-2 / rtol 1e-2), against the oracle in its
"exact" (all double) mode.  The reference's checker the oracle restates: test/infiniop/paged_attention.py:38-88;
its case list: test/infiniop/paged_attention.py:95-118.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import ATTN_TOL, assert_close, torch_to_bits
from infinicore_b200 import workloads

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF_LIB = ROOT / "oracle" / "_ref" / "lib" / "libinfiniop.so"


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    oracle.use_all_cores()
    yield _abi


def oracle_rows(d, rows=None):
    """Oracle output ("exact" mode) of the device-resident case `d`, for every sequence or for `rows`.
    For a subset the pages those sequences use are gathered into a compact pool first, so that a pool of
    tens of GB never has to cross to the host."""
    code = 12 if d.dtype == torch.float16 else 19
    if rows is None:
        return oracle.paged_attention(torch_to_bits(d.q), torch_to_bits(d.k_cache), torch_to_bits(d.v_cache),
                                      d.block_tables.cpu().numpy(), d.seq_lens.cpu().numpy(), d.scale, code)
    rows = torch.as_tensor(rows, device=d.q.device)
    lens = d.seq_lens[rows]
    pages = (lens + d.block_size - 1) // d.block_size
    tables = d.block_tables[rows]
    used = torch.cat([tables[i, :int(pages[i])] for i in range(len(rows))])
    compact = torch.zeros_like(tables)
    cursor = 0
    for i in range(len(rows)):
        n = int(pages[i])
        compact[i, :n] = torch.arange(cursor, cursor + n, device=tables.device)
        cursor += n
    return oracle.paged_attention(torch_to_bits(d.q[rows]), torch_to_bits(d.k_cache[used]), torch_to_bits(d.v_cache[used]),
                                  compact.cpu().numpy(), lens.cpu().numpy(), d.scale, code)


def reference_kernels(spec, tmp_path):
    """Output of the reference's own kernels (oracle/_ref, child process) on the inputs `spec` rebuilds."""
    env = dict(os.environ)
    env["INFINI_ROOT"] = str(REF_LIB.parent.parent)
    out = tmp_path / "ref.pt"
    res = subprocess.run([sys.executable, str(ROOT / "tests" / "ref_runner.py"), json.dumps(spec), str(out)],
                         env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    got = torch.load(out)
    assert "oracle/_ref" in got["library"]
    return got["out"]


def run(abi, d):
    """One attention call; returns (out, plan header of the streaming kernels as a dict)."""
    out = torch.zeros((d.num_seqs, d.num_heads, d.v_cache.shape[3]), dtype=d.dtype, device="cuda")
    op = abi.AttentionOp(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale)
    assert op.status == 0
    try:
        assert op.run(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens) == 0
        torch.cuda.synchronize()
        head = op.workspace.tensor[:32].cpu()
        plan = {"num_ranges": int(head[4:8].view(torch.int32)),
                "total_tiles": int(head[8:16].view(torch.int64)), "range_len": int(head[16:24].view(torch.int64))}
        assert abi.kernel_status() == 0, "a worker's bounded wait ran out"
    finally:
        op.destroy()
    return out, plan


def compare(d, got, want, what):
    atol, rtol = ATTN_TOL[d.dtype]
    assert_close(got.float().cpu().numpy(), want, atol, rtol, what)


needs_ref = pytest.mark.skipif(not REF_LIB.is_file(), reason="oracle/_ref not built")


# ---- configurations 2, 3, 4: one launch each, checked against the oracle and against the reference kernels ------

SPECS = {
    "c2": {"builder": "config2_llama8b", "kwargs": {"seed": 2, "device": "cuda"}, "caching": False},
    "c3": {"builder": "config3_ragged72b", "kwargs": {"seed": 3, "device": "cuda"}, "caching": False},
    "c4": {"builder": "config4_longctx", "kwargs": {"seed": 4, "device": "cuda"}, "caching": False},
}


def _launched(abi, name):
    spec = SPECS[name]
    d = getattr(workloads, spec["builder"])(**spec["kwargs"])
    got, plan = run(abi, d)
    return d, got, plan


@pytest.fixture(scope="module")
def config2(abi):
    yield _launched(abi, "c2")


@pytest.fixture(scope="module")
def config3(abi):
    yield _launched(abi, "c3")


@pytest.fixture(scope="module")
def config4(abi):
    yield _launched(abi, "c4")


def test_config2_every_sequence_against_the_oracle(config2):
    d, got, plan = config2
    assert d.num_seqs == 64 and d.total_tokens == 64 * 4096 and d.kv_bytes == 1073741824
    assert plan["total_tiles"] == 64 * 8 * 256
    compare(d, got, oracle_rows(d), "configuration 2, all 64 sequences")


@needs_ref
def test_config2_against_the_reference_kernels(config2, tmp_path):
    d, got, _ = config2
    compare(d, got, reference_kernels(SPECS["c2"], tmp_path).double().numpy(), "configuration 2 vs the reference kernels")


def test_config3_ragged_batch_against_the_oracle(config3):
    d, got, plan = config3
    lens = d.seq_lens.cpu()
    assert d.num_seqs == 256 and int(lens.min()) >= 16 and int(lens.max()) <= 32768 and int(lens.max()) > 16 * int(lens.min())
    # every worker streams the same number of tiles (+-1) whatever the mix of lengths
    assert plan["total_tiles"] == int(((lens + 15) // 16).sum()) * 8
    assert plan["num_ranges"] * plan["range_len"] - plan["total_tiles"] < plan["range_len"]
    compare(d, got, oracle_rows(d), "configuration 3, all 256 sequences")


@needs_ref
def test_config3_against_the_reference_kernels(config3, tmp_path):
    d, got, _ = config3
    compare(d, got, reference_kernels(SPECS["c3"], tmp_path).double().numpy(), "configuration 3 vs the reference kernels")


def test_config4_long_context_against_the_oracle(config4):
    d, got, plan = config4
    assert d.num_seqs == 2 and d.total_tokens == 2 * 131072 and d.dtype == torch.float16
    # 16 units (2 sequences x 8 kv-heads; the 4 q-heads of a group share one read) of 8192 tiles each are cut
    # into one range per resident warp: every output row is reduced over unit_tiles / range_len partial
    # records, every sequence's KV over 8 times as many pieces
    unit_tiles = 131072 // 16
    ways_per_unit = unit_tiles // plan["range_len"]
    assert plan["num_ranges"] >= 1024 and ways_per_unit >= 64 and 8 * ways_per_unit >= 128, plan
    compare(d, got, oracle_rows(d), "configuration 4, both sequences")


@needs_ref
def test_config4_against_the_reference_kernels(config4, tmp_path):
    d, got, _ = config4
    compare(d, got, reference_kernels(SPECS["c4"], tmp_path).double().numpy(), "configuration 4 vs the reference kernels")


# ---- configuration 5 ---------------------------------------------------------------------------------

def test_config5_rank0_shard_of_eight_against_the_oracle(abi):
    d = workloads.config5_shard(0, 8, device="cuda")
    lens = d.seq_lens.cpu()
    assert d.num_seqs == 256 and int(lens.min()) >= 1024 and int(lens.max()) <= 8192
    assert torch.equal(lens, workloads.config5_lengths()[0::8])
    got, _ = run(abi, d)
    compare(d, got, oracle_rows(d), "configuration 5, rank 0 of 8")


def test_config5_whole_batch_on_one_gpu_sampled_rows(abi):
    """All 2048 sequences on one GPU: more sequences than the in-kernel plan holds, so the plan comes from the
    separate plan kernel; 24 rows spread over the batch (first, last, shortest, longest among them) are checked."""
    d = workloads.config5_shard(0, 1, device="cuda")
    lens = d.seq_lens.cpu()
    assert d.num_seqs == 2048 and d.kv_bytes > 30e9
    got, plan = run(abi, d)
    assert plan["total_tiles"] == int(((lens + 15) // 16).sum()) * 8
    g = torch.Generator().manual_seed(55)
    rows = sorted(set([0, 2047, int(lens.argmin()), int(lens.argmax())] + torch.randperm(2048, generator=g)[:20].tolist()))
    compare(d, got[rows], oracle_rows(d, rows), "configuration 5, sampled rows of the whole batch")
    assert bool(torch.isfinite(got.float()).all())
