"""What the kernels report when a launch cannot do all of its work (infiniopGetKernelStatus).

Two situations, both made without faulting the GPU:
  * a worker's wait for one of its own TMA copies runs out.  The copy is withheld on purpose (a switch
    read when the descriptor is created makes worker 0 leave out the first copy it would issue, while it
    still expects the bytes), the wait limit is set to 20 ms, the kernel returns normally, the status word
    says WAIT_EXPIRED, and the next ordinary call on the same workspace is complete and correct;
  * with index checking on, block-table entries and cache slots outside the pool are reported and
    neutralised (read as block 0 / the row skipped) instead of touching foreign memory.
"""
import numpy as np
import pytest
import torch

import oracle
from helpers import ATTN_TOL, assert_close, torch_to_bits
from infinicore_b200 import workloads

pytestmark = pytest.mark.gpu

WAIT_EXPIRED, BLOCK_OUT_OF_RANGE, SLOT_OUT_OF_RANGE = 1, 2, 4


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def _oracle(case, lens=None):
    code = 12 if case.dtype == torch.float16 else 19
    return oracle.paged_attention(torch_to_bits(case.q), torch_to_bits(case.k_cache), torch_to_bits(case.v_cache),
                                  case.block_tables.numpy(), (case.seq_lens if lens is None else lens).numpy(), case.scale, code)


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_whole(abi):
    c = workloads.build_case("withheld", dtype=torch.bfloat16, seq_lens=[700, 33, 1500, 64], num_heads=32, num_kv_heads=8,
                             head_size=128, block_size=16, seed=81)
    d = c.to("cuda")
    want = _oracle(c)
    atol, rtol = ATTN_TOL[c.dtype]
    assert abi.kernel_status() == 0

    out = torch.full((4, 32, 128), 5.0, dtype=torch.bfloat16, device="cuda")
    got = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale, path="stream-withheld-copy", out=out)
    assert abi.kernel_status() == WAIT_EXPIRED
    assert abi.kernel_status() == 0, "reading the status clears it"
    # worker 0 owned the first tiles of sequence 0, kv-head 0: those rows are not to be trusted; every other
    # worker finished, so the sequences none of whose tiles were worker 0's are complete
    assert_close(got[1:].float().cpu().numpy(), want[1:], atol, rtol, "rows of the other workers")

    # the next ordinary call: complete and correct, nothing left behind
    out2 = torch.full((4, 32, 128), 5.0, dtype=torch.bfloat16, device="cuda")
    got2 = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale, path="stream", out=out2)
    assert abi.kernel_status() == 0
    assert_close(got2.float().cpu().numpy(), want, atol, rtol, "call after the expired wait")


@pytest.mark.parametrize("path", ["stream-checked", "generic-checked"])
def test_block_table_entries_outside_the_pool_are_reported(abi, path):
    c = workloads.build_case("badblock", dtype=torch.float16, seq_lens=[100, 40, 77], num_heads=8, num_kv_heads=2, head_size=64,
                             block_size=16, seed=82)
    d = c.to("cuda")
    atol, rtol = ATTN_TOL[c.dtype]
    # clean tables: nothing to report, results as ever
    got = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale, path=path)
    assert abi.kernel_status() == 0
    assert_close(got.float().cpu().numpy(), _oracle(c), atol, rtol, path)
    # the second page of sequence 1 points far outside the pool, the first page of sequence 2 is negative
    bad = d.block_tables.clone()
    bad[1, 1] = d.k_cache.shape[0] + 1000
    bad[2, 0] = -3
    got = abi.paged_attention(d.q, d.k_cache, d.v_cache, bad, d.seq_lens, d.scale, path=path)
    assert abi.kernel_status() == BLOCK_OUT_OF_RANGE
    assert bool(torch.isfinite(got.float()).all())
    # sequence 0 does not go through the bad entries
    assert_close(got[:1].float().cpu().numpy(), _oracle(c)[:1], atol, rtol, path + " untouched sequence")


def test_unchecked_descriptors_report_nothing_for_clean_inputs(abi):
    c = workloads.build_case("clean", dtype=torch.bfloat16, seq_lens=[300, 5], num_heads=8, num_kv_heads=8, head_size=128,
                             block_size=16, seed=83)
    d = c.to("cuda")
    abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale)
    abi.paged_caching(d.k_cache, d.v_cache, d.new_k, d.new_v, d.slot_mapping)
    assert abi.kernel_status() == 0


def test_slots_outside_the_pool_are_skipped_and_reported(abi):
    c = workloads.build_case("badslot", dtype=torch.float16, seq_lens=[20, 7, 33, 12], num_heads=4, num_kv_heads=2, head_size=64,
                             block_size=16, seed=84)
    d = c.to("cuda")
    slots = d.slot_mapping.clone()
    capacity = d.k_cache.shape[0] * 16
    slots[1] = capacity          # first slot past the pool
    slots[3] = capacity + 12345  # far past it
    before_k, before_v = d.k_cache.clone(), d.v_cache.clone()
    with abi.environment(INFINIOP_PAGED_CHECK_INDICES=1):
        abi.paged_caching(d.k_cache, d.v_cache, d.new_k, d.new_v, slots)
    assert abi.kernel_status() == SLOT_OUT_OF_RANGE
    # rows 0 and 2 landed, rows 1 and 3 went nowhere
    want_k, want_v = torch_to_bits(before_k).copy(), torch_to_bits(before_v).copy()
    ok = torch.tensor([0, 2])
    oracle.paged_caching(want_k, want_v, torch_to_bits(c.new_k[ok]), torch_to_bits(c.new_v[ok]), c.slot_mapping[ok].numpy())
    assert np.array_equal(torch_to_bits(d.k_cache), want_k) and np.array_equal(torch_to_bits(d.v_cache), want_v)


def test_python_operator_reads_the_same_word():
    import infinicore_b200 as ib

    assert ib.kernel_status() == 0
