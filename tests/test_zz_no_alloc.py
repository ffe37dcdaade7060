"""infiniopPagedAttentionStaticWorkspace - the entry point for callers that cannot allocate.

Some users of this library have no device memory to offer as workspace: a serving engine that gave
all free HBM to its KV pool, a process whose allocator is frozen once serving starts, an operator
callback that may only touch buffers its host framework registered.  For them the library carries
a 32 MiB scratch array of its own.  This test calls that entry point through the C ABI - passing
inputs and outputs only - and checks the result against the regular infiniopPagedAttention (caller
workspace) and against the CPU oracle on two different problems in a row, so that whatever the first
call left in the shared array is in place when the second one runs; that calls after the first leave
the device's free memory untouched (the first is the one on which the CUDA runtime places the array);
that the other kernel routes (wide heads, the generic kernel without workspace, the separate plan
kernel) work on the shared array too; and that a problem too large for the array is refused before
anything is launched.

Collected last on purpose: the file name sorts after every other test file.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from helpers import ATTN_TOL, assert_close, torch_to_bits
from infinicore_b200 import workloads

pytestmark = pytest.mark.gpu

STATIC_BYTES = 32 << 20


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def _static_call(abi, d, out, path=None, check_memory=False):
    """Creates a descriptor, runs the static-workspace entry point, returns (status, workspace need).
    With check_memory the device's free memory is read right before and right after the call (everything
    the test itself allocates exists by then): the call must not have taken a byte."""
    from infinicore_b200.libinfiniop import LIBINFINIOP

    op = abi.AttentionOp(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale, path=path)
    assert op.status == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    status = LIBINFINIOP.infiniopPagedAttentionStaticWorkspace(
        op.desc, out.data_ptr(), d.q.data_ptr(), d.k_cache.data_ptr(), d.v_cache.data_ptr(),
        d.block_tables.data_ptr(), d.seq_lens.data_ptr(), None, None)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    if check_memory:
        assert free_after == free_before, f"the call changed the device's free memory by {free_before - free_after} bytes"
    need = op.workspace_size
    op.destroy()
    return status, need


def _oracle(case):
    code = 12 if case.dtype == torch.float16 else 19
    return oracle.paged_attention(torch_to_bits(case.q), torch_to_bits(case.k_cache), torch_to_bits(case.v_cache),
                                  case.block_tables.numpy(), case.seq_lens.numpy(), case.scale, code)


def test_two_calls_in_a_row_match_the_regular_entry_point_and_the_oracle(abi):
    cases = [
        workloads.build_case("static_a", dtype=torch.bfloat16, seq_lens=[2048, 777, 16, 1500, 3000, 1, 640, 2047],
                             num_heads=32, num_kv_heads=8, head_size=128, block_size=16, seed=71),
        workloads.build_case("static_b", dtype=torch.bfloat16, seq_lens=[5, 4096, 300, 33, 1024, 2000, 64, 129],
                             num_heads=32, num_kv_heads=8, head_size=128, block_size=16, seed=72),
    ]
    atol, rtol = ATTN_TOL[torch.bfloat16]
    for i, case in enumerate(cases):
        d = case.to("cuda")
        want = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale)
        got = torch.zeros_like(want)
        # the first call on a device is the one that makes the runtime place the array; from the second on
        # the device's free memory must not move
        status, need = _static_call(abi, d, got, check_memory=(i > 0))
        assert status == 0
        assert 0 < need <= STATIC_BYTES, "the case is meant to use the built-in scratch"
        assert_close(got.float().cpu().numpy(), want.float().cpu().numpy(), atol, rtol, case.name + " vs the regular entry point")
        assert_close(got.float().cpu().numpy(), _oracle(case), atol, rtol, case.name + " vs the oracle")
        assert bool(torch.isfinite(got.float()).all())


# Other users of the shared array: each runs right after a call of a DIFFERENT shape has left its plan,
# tasks and records in it, so anything a kernel wrongly expects to find zeroed (or its own) would show.
OTHER_ROUTES = [
    # key width 576, value width 512 (latent attention): the four-warp wide-head kernel, plan from the plan kernel
    ("wide_576_512", dict(dtype=torch.bfloat16, seq_lens=[300, 17, 1025], num_heads=16, num_kv_heads=1, head_size=576,
                          value_size=512, block_size=16, seed=74), None),
    # block size 8: the generic kernel, which needs no workspace at all (scratch pointer null, size 0)
    ("generic_bs8", dict(dtype=torch.float16, seq_lens=[50, 9, 120], num_heads=4, num_kv_heads=2, head_size=64,
                         block_size=8, seed=75), None),
    # the plan computed by the separate one-CTA kernel instead of inside the main kernel
    ("plan_kernel", dict(dtype=torch.float16, seq_lens=[700, 64, 2000, 1, 333], num_heads=8, num_kv_heads=2, head_size=64,
                         block_size=16, seed=76), "stream-plan-kernel"),
]


@pytest.mark.parametrize("name,kwargs,path", OTHER_ROUTES, ids=[r[0] for r in OTHER_ROUTES])
def test_other_kernel_routes_share_the_array(abi, name, kwargs, path):
    stale = workloads.build_case("static_stale", dtype=torch.bfloat16, seq_lens=[1000, 50, 3000, 7], num_heads=32, num_kv_heads=8,
                                 head_size=128, block_size=16, seed=77).to("cuda")
    scratch_out = torch.zeros((4, 32, 128), dtype=torch.bfloat16, device="cuda")

    case = workloads.build_case(name, **kwargs)
    d = case.to("cuda")
    # the regular entry point first: the CUDA runtime loads a kernel's code (which takes device memory) on
    # its first launch in the process, and that is not what the memory check below is about
    regular = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale, path=path)
    assert _static_call(abi, stale, scratch_out)[0] == 0
    got = torch.zeros((d.num_seqs, d.num_heads, d.v_cache.shape[3]), dtype=d.dtype, device="cuda")
    status, need = _static_call(abi, d, got, path=path, check_memory=True)
    assert torch.equal(got.view(torch.int16), regular.view(torch.int16)), "differs from the regular entry point"
    assert status == 0 and need <= STATIC_BYTES
    if name == "generic_bs8":
        assert need == 0
    atol, rtol = ATTN_TOL[case.dtype]
    assert_close(got.float().cpu().numpy(), _oracle(case), atol, rtol, name + " vs the oracle")


def test_a_problem_larger_than_the_array_is_refused_untouched(abi):
    # 2048 sequences x 8 kv-heads of records do not fit in 32 MiB; shapes alone decide, so tiny pools do
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
