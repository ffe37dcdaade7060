"""infiniopPagedAttentionStaticWorkspace - the entry point for callers that cannot allocate.

Some users of this library have no device memory to offer as workspace: a serving engine that gave
all free HBM to its KV pool, a process whose allocator is frozen once serving starts, an operator
callback that may only touch buffers its host framework registered.  For them the library carries
a 16 MiB scratch array of its own.  This test calls that entry point through the C ABI - passing
inputs and outputs only - and checks the result against the regular infiniopPagedAttention (caller
workspace) on two different problems in a row, so that whatever the first call left in the shared
array is in place when the second one runs.  It also checks that a problem too large for the array
is refused before anything is launched.

Collected last on purpose: the file name sorts after every other test file.
"""
import ctypes

import pytest
import torch

from helpers import ATTN_TOL, assert_close
from infinicore_b200 import workloads

pytestmark = pytest.mark.gpu

STATIC_BYTES = 16 << 20


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def _static_call(abi, d, out):
    """Creates a descriptor, runs the static-workspace entry point, returns (status, workspace need)."""
    from infinicore_b200.libinfiniop import LIBINFINIOP

    op = abi.AttentionOp(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale)
    assert op.status == 0
    status = LIBINFINIOP.infiniopPagedAttentionStaticWorkspace(
        op.desc, out.data_ptr(), d.q.data_ptr(), d.k_cache.data_ptr(), d.v_cache.data_ptr(),
        d.block_tables.data_ptr(), d.seq_lens.data_ptr(), None, None)
    torch.cuda.synchronize()
    need = op.workspace_size
    op.destroy()
    return status, need


def test_two_calls_in_a_row_match_the_regular_entry_point(abi):
    cases = [
        workloads.build_case("static_a", dtype=torch.bfloat16, seq_lens=[2048, 777, 16, 1500, 3000, 1, 640, 2047],
                             num_heads=32, num_kv_heads=8, head_size=128, block_size=16, seed=71),
        workloads.build_case("static_b", dtype=torch.bfloat16, seq_lens=[5, 4096, 300, 33, 1024, 2000, 64, 129],
                             num_heads=32, num_kv_heads=8, head_size=128, block_size=16, seed=72),
    ]
    atol, rtol = ATTN_TOL[torch.bfloat16]
    for case in cases:
        d = case.to("cuda")
        want = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale)
        got = torch.zeros_like(want)
        status, need = _static_call(abi, d, got)
        assert status == 0
        assert 0 < need <= STATIC_BYTES, "the case is meant to use the built-in scratch"
        assert_close(got.float().cpu().numpy(), want.float().cpu().numpy(), atol, rtol, case.name)
        assert bool(torch.isfinite(got.float()).all())


def test_a_problem_larger_than_the_array_is_refused_untouched(abi):
    # 2048 sequences x 8 kv-heads of records do not fit in 16 MiB; shapes alone decide, so tiny pools do
    c = workloads.build_case("static_big", dtype=torch.float16, seq_lens=[1] * 2048, num_heads=32, num_kv_heads=8,
                             head_size=128, block_size=16, seed=73)
    d = c.to("cuda")
    out = torch.full((2048, 32, 128), 4.0, dtype=torch.float16, device="cuda")
    status, need = _static_call(abi, d, out)
    assert need > STATIC_BYTES
    assert status == 13  # INFINI_STATUS_INSUFFICIENT_WORKSPACE
    assert bool((out == 4.0).all())


def test_null_descriptor_is_reported(abi):
    from infinicore_b200.libinfiniop import LIBINFINIOP

    assert LIBINFINIOP.infiniopPagedAttentionStaticWorkspace(None, None, None, None, None, None, None, None, None) == 4
