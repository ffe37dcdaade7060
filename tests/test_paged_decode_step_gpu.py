"""GPU parity of infiniopPagedDecodeStep (append the newest K/V row, then attend) through the C ABI.

The operator has no reference counterpart; what it must equal is the reference's pair of calls.  So
every case is checked three ways: the caches after the call are bit-exact against the oracle's
paged_caching with the slots the block tables name; the output is within the decode tolerance
(fp16 2e-3 / 2e-3, bf16 1e-2 / 1e-2) of the oracle's attention over those caches; and the result
matches infiniopPagedCaching followed by infiniopPagedAttention on a second copy of the inputs.
Both routes are covered: the streaming kernel that takes the rows itself, and the generic path
(append kernel + attention kernel)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import ATTN_TOL, assert_close, torch_to_bits
from infinicore_b200 import workloads
from infinicore_b200.libinfiniop import InfiniDtype

pytestmark = pytest.mark.gpu

PATHS = [None, "generic", "stream-plan-kernel", "stream-3x4", "stream-pool"]


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def run_and_check(abi, c, path, alibi=None, index_dtype=None, poison=False):
    d = c.to("cuda")
    if poison:
        # the slots that receive the new rows hold NaN before the call: nothing of them may reach the output
        nan = torch.tensor(float("nan"), dtype=c.dtype, device="cuda")
        for i, slot in enumerate(c.slot_mapping.tolist()):
            if slot >= 0:
                d.k_cache[slot // c.block_size, :, slot % c.block_size, :] = nan
                d.v_cache[slot // c.block_size, :, slot % c.block_size, :] = nan
    k0, v0 = d.k_cache.clone(), d.v_cache.clone()
    bt, lens = d.block_tables, d.seq_lens
    if index_dtype is not None:
        bt, lens = bt.to(index_dtype), lens.to(index_dtype)
    out = torch.full((c.q.shape[0], c.num_heads, c.v_cache.shape[3]), 7.0, dtype=c.dtype, device="cuda")
    dt_code = InfiniDtype.I32 if index_dtype == torch.int32 else None
    got = abi.paged_decode_step(d.q, d.k_cache, d.v_cache, d.new_k, d.new_v, bt, lens, d.scale,
                                alibi.cuda() if alibi is not None else None, path=path, out=out, index_dtype=dt_code)

    # (1) caches: bit-exact against the oracle's scatter
    kb, vb = torch_to_bits(k0), torch_to_bits(v0)
    oracle.paged_caching(kb, vb, torch_to_bits(c.new_k), torch_to_bits(c.new_v), c.slot_mapping.numpy())
    assert np.array_equal(torch_to_bits(d.k_cache), kb), "k_cache differs from the oracle's scatter"
    assert np.array_equal(torch_to_bits(d.v_cache), vb), "v_cache differs from the oracle's scatter"
    # (2) output: the oracle's attention over the updated caches
    dt = 12 if c.dtype == torch.float16 else 19
    want = oracle.paged_attention(torch_to_bits(c.q), kb, vb, c.block_tables.numpy(), c.seq_lens.numpy(), c.scale, dt,
                                  alibi.numpy() if alibi is not None else None)
    live = (c.seq_lens > 0).numpy()
    atol, rtol = ATTN_TOL[c.dtype]
    assert_close(got.float().cpu().numpy()[live], want[live], atol, rtol, c.name)
    assert bool((got[~torch.from_numpy(live)] == 7.0).all()), "rows of empty sequences must stay untouched"
    # (3) the reference's pair of calls on the same inputs
    abi.paged_caching(k0, v0, d.new_k, d.new_v, d.slot_mapping)
    pair = abi.paged_attention(d.q, k0, v0, bt, lens, d.scale, alibi.cuda() if alibi is not None else None, path=path,
                               index_dtype=dt_code)
    assert torch.equal(k0, d.k_cache) and torch.equal(v0, d.v_cache)
    assert_close(got.float().cpu().numpy()[live], pair.float().cpu().numpy()[live], atol, rtol, c.name + " vs pair of calls")
    return got


@pytest.mark.parametrize("path", PATHS)
def test_config1_flow(abi, path):
    run_and_check(abi, workloads.config1_small(seed=1), path)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype,heads,kvh,hd,bs", [(torch.bfloat16, 32, 8, 128, 16), (torch.float16, 8, 2, 64, 16),
                                                   (torch.bfloat16, 32, 1, 128, 32), (torch.float16, 12, 1, 128, 16),
                                                   (torch.bfloat16, 16, 2, 256, 16)])
def test_every_row_of_the_last_page(abi, path, dtype, heads, kvh, hd, bs):
    """Lengths 1..2*block+1: the newest token lands on every row of a page, on both sides of a page
    boundary and of a 16-token tile boundary; group sizes 4, 8, 12 and 32 (several head tiles share one
    kv-head, only one of them stores the row); the destination slots hold NaN beforehand."""
    lens = list(range(1, 2 * bs + 2)) + [0, 5 * bs, 5 * bs + 1]
    c = workloads.build_case("lastpage", dtype=dtype, seq_lens=lens, num_heads=heads, num_kv_heads=kvh, head_size=hd,
                             block_size=bs, seed=41, slack_blocks=3)
    run_and_check(abi, c, path, poison=True)


@pytest.mark.parametrize("path", [None, "generic"])
def test_ragged_long_batch_with_alibi_and_int32_indices(abi, path):
    lens = workloads.config3_lengths(seed=7, num_seqs=48, hi=6000)
    c = workloads.build_case("ragged", dtype=torch.bfloat16, seq_lens=lens, num_heads=16, num_kv_heads=4, head_size=128,
                             block_size=16, seed=42, std=0.5)
    alibi = -torch.linspace(0.01, 0.3, 16, dtype=torch.float32)
    run_and_check(abi, c, path, alibi=alibi, index_dtype=torch.int32, poison=True)


def test_shapes_the_streaming_kernel_does_not_take_use_the_append_kernel(abi):
    """Block size 4 (no streaming plan) and the 576/512 latent-attention shape: append kernel + generic attention."""
    c = workloads.build_case("bs4", dtype=torch.float16, seq_lens=[1, 4, 5, 23, 0, 64], num_heads=4, num_kv_heads=2, head_size=64,
                             block_size=4, seed=43)
    run_and_check(abi, c, None, poison=True)
    c = workloads.build_case("mla", dtype=torch.bfloat16, seq_lens=[17, 1, 90], num_heads=8, num_kv_heads=1, head_size=576,
                             block_size=16, seed=44, value_size=512, std=0.3)
    run_and_check(abi, c, None)


@pytest.mark.parametrize("value", [576, 512])
def test_wide_heads_take_the_rows_inside_the_kernel(abi, value):
    """Key width 576 on the four-warp kernel: every warp swaps the new row into what it reads, the
    stores into the cache are shared out; lengths on every row of a page; 3 head tiles per kv-head."""
    lens = list(range(1, 35)) + [0, 400, 1000]
    c = workloads.build_case("wide_step", dtype=torch.bfloat16, seq_lens=lens, num_heads=20, num_kv_heads=1, head_size=576,
                             value_size=value, block_size=16, seed=48, std=0.3, slack_blocks=3)
    run_and_check(abi, c, None, poison=True)


def test_unaligned_new_rows_fall_back_to_the_append_kernel(abi):
    """new_k / new_v views whose rows are not 16-byte aligned: same results through the unfused route."""
    c = workloads.build_case("unaligned", dtype=torch.bfloat16, seq_lens=[33, 16, 100], num_heads=8, num_kv_heads=2, head_size=128,
                             block_size=16, seed=45)
    pad_k = torch.zeros(c.new_k.numel() + 1, dtype=c.dtype)
    pad_v = torch.zeros(c.new_v.numel() + 1, dtype=c.dtype)
    pad_k[1:] = c.new_k.flatten()
    pad_v[1:] = c.new_v.flatten()

    class Shifted:  # the case with new rows living 2 bytes off a 16-byte boundary on the device
        def __init__(self, base):
            self.__dict__.update(base.__dict__)

        def to(self, device):
            d = c.to(device)
            d.new_k = pad_k.to(device)[1:].view_as(c.new_k)
            d.new_v = pad_v.to(device)[1:].view_as(c.new_v)
            return d

    run_and_check(abi, Shifted(c), None)


def test_descriptor_refuses_bad_new_rows(abi):
    from infinicore_b200.libinfiniop import InfiniStatusError

    c = workloads.build_case("bad", dtype=torch.float16, seq_lens=[8, 9], num_heads=4, num_kv_heads=2, head_size=64, block_size=16, seed=46)
    d = c.to("cuda")
    out = torch.zeros_like(d.q)
    for bad_k, code in [(d.new_k[:1], 11), (d.new_k.float(), 10), (torch.zeros((2, 2, 128), dtype=c.dtype, device="cuda")[:, :, ::2], 12),
                        (torch.zeros((2, 4, 64), dtype=c.dtype, device="cuda")[:, ::2], 12)]:
        op = abi.DecodeStepOp(out, d.q, d.k_cache, d.v_cache, bad_k, d.new_v, d.block_tables, d.seq_lens, None, d.scale)
        assert op.status == code, (tuple(bad_k.shape), op.status)
    with pytest.raises(InfiniStatusError):
        abi.check_error(abi.LIBINFINIOP.infiniopGetPagedDecodeStepWorkspaceSize(None, None))


def test_python_operator_and_two_steps_in_a_row(abi):
    """infinicore_b200.paged_decode_step: two consecutive decode steps of growing sequences."""
    import infinicore_b200 as ib

    c = workloads.build_case("steps", dtype=torch.bfloat16, seq_lens=[15, 14, 30, 200], num_heads=32, num_kv_heads=8, head_size=128,
                             block_size=16, seed=47, slack_blocks=0, max_blocks_per_seq=14)
    d = c.to("cuda")
    kb, vb = torch_to_bits(c.k_cache).copy(), torch_to_bits(c.v_cache).copy()
    lens = c.seq_lens.clone()
    gen = torch.Generator().manual_seed(5)
    for step in range(2):
        nk = torch.randn(c.new_k.shape, generator=gen).to(c.dtype)
        nv = torch.randn(c.new_v.shape, generator=gen).to(c.dtype)
        q = torch.randn(c.q.shape, generator=gen).to(c.dtype)
        slots = torch.tensor([int(c.block_tables[i, (int(lens[i]) - 1) // 16]) * 16 + (int(lens[i]) - 1) % 16 for i in range(4)])
        got = ib.paged_decode_step(q.cuda(), d.k_cache, d.v_cache, nk.cuda(), nv.cuda(), d.block_tables, lens.cuda(), None, c.scale)
        torch.cuda.synchronize()
        oracle.paged_caching(kb, vb, torch_to_bits(nk), torch_to_bits(nv), slots.numpy())
        want = oracle.paged_attention(torch_to_bits(q), kb, vb, c.block_tables.numpy(), lens.numpy(), c.scale, 19)
        assert np.array_equal(torch_to_bits(d.k_cache), kb)
        atol, rtol = ATTN_TOL[c.dtype]
        assert_close(got.float().cpu().numpy(), want, atol, rtol, f"step {step}")
        lens = lens + 1  # stays inside each sequence's last allocated page for these lengths


# ---- the RoPE form: rotate q and the new K row, append, attend ---------------------------------------


def rope_tables(table_len, dhead, dtype, theta=1e4):
    freqs = 1.0 / (theta ** (torch.arange(0, dhead, 2)[: dhead // 2].float() / dhead))
    angles = torch.outer(torch.arange(table_len).float(), freqs)
    return torch.sin(angles).to(dtype), torch.cos(angles).to(dtype)


def run_and_check_rope(abi, c, path, algo, alibi=None, pos_ids=None, table_len=None, q_view=None):
    """Checks infiniopPagedDecodeStepRoPE against the oracle's rope -> caching -> attention (caches bit-exact,
    output within the decode tolerance) and against the four separate calls of this library."""
    d = c.to("cuda")
    nan = torch.tensor(float("nan"), dtype=c.dtype, device="cuda")
    for slot in c.slot_mapping.tolist():
        if slot >= 0:
            d.k_cache[slot // c.block_size, :, slot % c.block_size, :] = nan
            d.v_cache[slot // c.block_size, :, slot % c.block_size, :] = nan
    k0, v0 = d.k_cache.clone(), d.v_cache.clone()
    # the position of the new token is its index in the sequence
    pos = (c.seq_lens - 1).clamp(min=0) if pos_ids is None else pos_ids
    table_len = int(pos.max()) + 1 if table_len is None else table_len
    sin, cos = rope_tables(table_len, c.head_size, c.dtype)
    q_dev = d.q if q_view is None else q_view(d.q)
    q_before, nk_before = q_dev.clone(), d.new_k.clone()
    out = torch.full((c.q.shape[0], c.num_heads, c.v_cache.shape[3]), 7.0, dtype=c.dtype, device="cuda")
    got = abi.paged_decode_step_rope(q_dev, d.k_cache, d.v_cache, d.new_k, d.new_v, d.block_tables, d.seq_lens, d.scale,
                                     pos.cuda(), sin.cuda(), cos.cuda(), algo,
                                     alibi.cuda() if alibi is not None else None, path=path, out=out)
    assert torch.equal(q_dev, q_before) and torch.equal(d.new_k, nk_before), "q / new_k must stay as they were"

    dt = 12 if c.dtype == torch.float16 else 19
    q_rot = oracle.rope(torch_to_bits(c.q), pos.numpy(), torch_to_bits(sin), torch_to_bits(cos), dt, algo == 0)
    k_rot = oracle.rope(torch_to_bits(c.new_k), pos.numpy(), torch_to_bits(sin), torch_to_bits(cos), dt, algo == 0)
    kb, vb = torch_to_bits(k0), torch_to_bits(v0)
    oracle.paged_caching(kb, vb, k_rot, torch_to_bits(c.new_v), c.slot_mapping.numpy())
    assert np.array_equal(torch_to_bits(d.k_cache), kb), "k_cache differs from the oracle's rotated scatter"
    assert np.array_equal(torch_to_bits(d.v_cache), vb), "v_cache differs from the oracle's scatter"
    want = oracle.paged_attention(q_rot, kb, vb, c.block_tables.numpy(), c.seq_lens.numpy(), c.scale, dt,
                                  alibi.numpy() if alibi is not None else None)
    live = (c.seq_lens > 0).numpy()
    atol, rtol = ATTN_TOL[c.dtype]
    assert_close(got.float().cpu().numpy()[live], want[live], atol, rtol, c.name)
    assert bool((got[~torch.from_numpy(live)] == 7.0).all()), "rows of empty sequences must stay untouched"

    # the four calls a decode layer of the reference issues
    q2 = abi.rope(q_dev, pos.cuda(), sin.cuda(), cos.cuda(), algo)
    nk2 = abi.rope(d.new_k, pos.cuda(), sin.cuda(), cos.cuda(), algo)
    assert np.array_equal(torch_to_bits(q2), q_rot) and np.array_equal(torch_to_bits(nk2), k_rot)
    abi.paged_caching(k0, v0, nk2, d.new_v, d.slot_mapping)
    four = abi.paged_attention(q2, k0, v0, d.block_tables, d.seq_lens, d.scale, alibi.cuda() if alibi is not None else None, path=path)
    assert torch.equal(k0, d.k_cache) and torch.equal(v0, d.v_cache)
    assert_close(got.float().cpu().numpy()[live], four.float().cpu().numpy()[live], atol, rtol, c.name + " vs four calls")


@pytest.mark.parametrize("algo", [0, 1])
@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype,heads,kvh,hd,bs", [(torch.bfloat16, 32, 8, 128, 16), (torch.float16, 8, 2, 64, 16),
                                                   (torch.float16, 12, 1, 128, 32), (torch.bfloat16, 16, 2, 256, 16)])
def test_rope_form_on_every_row_of_the_last_page(abi, path, algo, dtype, heads, kvh, hd, bs):
    lens = list(range(1, 2 * bs + 2)) + [0, 5 * bs, 5 * bs + 1]
    c = workloads.build_case("rope_lastpage", dtype=dtype, seq_lens=lens, num_heads=heads, num_kv_heads=kvh, head_size=hd,
                             block_size=bs, seed=51, slack_blocks=3)
    run_and_check_rope(abi, c, path, algo)


@pytest.mark.parametrize("path", [None, "generic"])
def test_rope_form_ragged_long_batch_with_alibi(abi, path):
    lens = workloads.config3_lengths(seed=9, num_seqs=40, hi=5000)
    c = workloads.build_case("rope_ragged", dtype=torch.bfloat16, seq_lens=lens, num_heads=16, num_kv_heads=4, head_size=128,
                             block_size=16, seed=52, std=0.5)
    alibi = -torch.linspace(0.01, 0.3, 16, dtype=torch.float32)
    run_and_check_rope(abi, c, path, 1, alibi=alibi)


def test_rope_form_positions_outside_the_tables_and_strided_q(abi):
    """Position ids beyond the tables leave their rows unrotated; q as a view with padded rows (the rotated
    copy the attention reads is dense whatever q's strides are)."""
    c = workloads.build_case("rope_edge", dtype=torch.float16, seq_lens=[40, 3, 17, 64], num_heads=8, num_kv_heads=2, head_size=64,
                             block_size=16, seed=53)
    pos = torch.tensor([39, 100, -2, 5], dtype=torch.int64)

    def padded(q):
        base = torch.zeros((q.shape[0], q.shape[1], q.shape[2] + 8), dtype=q.dtype, device=q.device)
        base[:, :, : q.shape[2]] = q
        return base[:, :, : q.shape[2]]

    run_and_check_rope(abi, c, None, 1, pos_ids=pos, table_len=64, q_view=padded)
    run_and_check_rope(abi, c, "generic", 0, pos_ids=pos, table_len=64, q_view=padded)


def test_rope_form_without_a_streaming_plan(abi):
    """Block size 4: rotation kernel, append kernel, generic attention; the workspace holds only the rotated rows."""
    c = workloads.build_case("rope_bs4", dtype=torch.bfloat16, seq_lens=[1, 4, 5, 23, 0, 64], num_heads=4, num_kv_heads=2, head_size=64,
                             block_size=4, seed=54)
    run_and_check_rope(abi, c, None, 1)


def test_rope_form_python_operator(abi):
    import infinicore_b200 as ib

    c = workloads.build_case("rope_py", dtype=torch.bfloat16, seq_lens=[15, 14, 30, 200], num_heads=32, num_kv_heads=8, head_size=128,
                             block_size=16, seed=55)
    d = c.to("cuda")
    pos = c.seq_lens - 1
    sin, cos = rope_tables(256, 128, c.dtype)
    k0, v0 = d.k_cache.clone(), d.v_cache.clone()
    got = ib.paged_decode_step(d.q, d.k_cache, d.v_cache, d.new_k, d.new_v, d.block_tables, d.seq_lens, None, c.scale,
                               pos_ids=pos.cuda(), sin_table=sin.cuda(), cos_table=cos.cuda(), rope_algo=ib.RopeAlgo.GPT_NEOX)
    q2 = ib.rope(d.q, pos.cuda(), sin.cuda(), cos.cuda(), ib.RopeAlgo.GPT_NEOX)
    nk2 = ib.rope(d.new_k, pos.cuda(), sin.cuda(), cos.cuda())
    ib.paged_caching(k0, v0, nk2, d.new_v, d.slot_mapping)
    want = ib.paged_attention(q2, k0, v0, d.block_tables, d.seq_lens, None, c.scale)
    torch.cuda.synchronize()
    assert torch.equal(k0, d.k_cache) and torch.equal(v0, d.v_cache)
    atol, rtol = ATTN_TOL[c.dtype]
    assert_close(got.float().cpu().numpy(), want.float().cpu().numpy(), atol, rtol, "python rope step")


def test_rope_form_refuses_bad_tables(abi):
    c = workloads.build_case("rope_bad", dtype=torch.float16, seq_lens=[8, 9], num_heads=4, num_kv_heads=2, head_size=64, block_size=16, seed=56)
    d = c.to("cuda")
    sin, cos = (t.cuda() for t in rope_tables(16, 64, c.dtype))
    pos = torch.tensor([7, 8], device="cuda")
    from infinicore_b200.libinfiniop import InfiniStatusError

    for bad_pos, bad_sin, code in [(pos.float(), sin, 10), (pos[:1], sin, 11), (pos, sin[:, :16], 11), (pos, sin.to(torch.bfloat16), 10),
                                   (pos, sin.t().contiguous().t(), 12)]:
        with pytest.raises(InfiniStatusError) as err:
            abi.paged_decode_step_rope(d.q, d.k_cache, d.v_cache, d.new_k, d.new_v, d.block_tables, d.seq_lens, d.scale,
                                       bad_pos, bad_sin, bad_sin if bad_sin.shape != sin.shape or bad_sin.dtype != sin.dtype else cos, 1)
        assert err.value.status == code


@pytest.mark.parametrize("fuse", [None, "1", "0"])
def test_large_batches_take_the_append_kernel_unless_told_otherwise(abi, fuse, monkeypatch):
    """More units (sequence x kv-head x head tile) than workers: by default the rows go through the append
    kernel; INFINIOP_PAGED_DECODE_STEP_FUSE = 1 hands them to the attention kernel all the same, 0 never does.
    Every route gives the same caches and outputs."""
    if fuse is None:
        monkeypatch.delenv("INFINIOP_PAGED_DECODE_STEP_FUSE", raising=False)
    else:
        monkeypatch.setenv("INFINIOP_PAGED_DECODE_STEP_FUSE", fuse)
    gen = torch.Generator().manual_seed(57)
    lens = torch.randint(1, 200, (320,), generator=gen).tolist()
    c = workloads.build_case("many", dtype=torch.bfloat16, seq_lens=lens, num_heads=32, num_kv_heads=8, head_size=128,
                             block_size=16, seed=58)
    run_and_check(abi, c, None, poison=True)
    run_and_check_rope(abi, c, None, 1)


@pytest.mark.parametrize("path", [None, "generic"])
@pytest.mark.parametrize("name", ["layer_bf16_gqa4_hd128_neox", "layer_fp16_gqa2_hd64_gptj"])
def test_rope_form_against_the_reference_checkers_chained(abi, name, path):
    """infiniopPagedDecodeStepRoPE against golden files made by chaining the reference's own checkers (rotary
    embedding of q and new K, cache scatter, attention): caches bit for bit, output within the decode tolerance."""
    from helpers import bits_to_float, bits_to_torch, load_golden

    g = load_golden(name)
    dt = int(g["dtype"])
    t = {k: bits_to_torch(g[k], dt).cuda() for k in ("q", "k_cache", "v_cache", "new_k", "new_v", "sin_table", "cos_table")}
    idx = {k: torch.from_numpy(g[k]).cuda() for k in ("block_tables", "seq_lens", "pos_ids")}
    got = abi.paged_decode_step_rope(t["q"], t["k_cache"], t["v_cache"], t["new_k"], t["new_v"], idx["block_tables"], idx["seq_lens"],
                                     float(g["scale"]), idx["pos_ids"], t["sin_table"], t["cos_table"], int(g["algo"]), path=path)
    assert np.array_equal(torch_to_bits(t["k_cache"]), g["k_cache_after"])
    assert np.array_equal(torch_to_bits(t["v_cache"]), g["v_cache_after"])
    atol, rtol = ATTN_TOL[dt]
    assert_close(got.float().cpu().numpy(), bits_to_float(g["out"], dt), atol, rtol, name)
