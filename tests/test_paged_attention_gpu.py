"""GPU parity of infiniopPagedAttention through the C ABI.

Checked against (a) the reference's golden outputs, (b) the CPU oracle in "exact" mode on the same
seeded inputs, at the parity tolerance of the path: fp16 atol 2e-3 / rtol 2e-3, bf16 atol 1e-2 /
rtol 1e-2.  Both kernels are covered: the streaming TMA/MMA path (default where eligible) and the
generic path (forced with INFINIOP_PAGED_DECODE_PATH=generic at descriptor creation)."""
import math

import numpy as np
import pytest
import torch

import oracle
from helpers import ATTN_TOL, TORCH_DTYPE, assert_close, bits_to_float, bits_to_torch, golden_names, load_golden, torch_to_bits
from infinicore_b200 import workloads

pytestmark = pytest.mark.gpu

PATHS = [None, "generic"]


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def oracle_out(case, alibi=None, seq_lens=None, mode="exact"):
    dt = 12 if case.dtype == torch.float16 else 19
    lens = case.seq_lens if seq_lens is None else seq_lens
    return oracle.paged_attention(
        torch_to_bits(case.q), torch_to_bits(case.k_cache), torch_to_bits(case.v_cache),
        case.block_tables.cpu().numpy(), lens.cpu().numpy(), case.scale, dt,
        alibi.cpu().numpy() if alibi is not None else None, mode=mode)


def run_case(abi, case, path, alibi=None, index_dtype=None, seq_lens=None, out=None):
    d = case.to("cuda")
    lens = d.seq_lens if seq_lens is None else seq_lens.cuda()
    bt = d.block_tables
    if index_dtype is not None:
        bt, lens = bt.to(torch.int32), lens.to(torch.int32)
    return abi.paged_attention(d.q, d.k_cache, d.v_cache, bt, lens, d.scale,
                               alibi.cuda() if alibi is not None else None, path=path, out=out, index_dtype=index_dtype)


def check(case, got, want):
    atol, rtol = ATTN_TOL[case.dtype]
    assert_close(got.float().cpu().numpy(), want, atol, rtol, case.name)


# ---- golden vectors produced by the reference's own checker -------------------------------------

@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("name", golden_names("attn_"))
def test_golden(abi, name, path):
    g = load_golden(name)
    dt = int(g["dtype"])
    dev = "cuda"
    q, kc, vc = (bits_to_torch(g[k], dt).to(dev) for k in ("q", "k_cache", "v_cache"))
    alibi = torch.from_numpy(g["alibi"]).to(dev) if g["alibi"].size else None
    got = abi.paged_attention(q, kc, vc, torch.from_numpy(g["block_tables"]).to(dev),
                              torch.from_numpy(g["seq_lens"]).to(dev), float(g["scale"]), alibi, path=path)
    atol, rtol = ATTN_TOL[dt]
    assert_close(got.float().cpu().numpy(), bits_to_float(g["out"], dt), atol, rtol, f"{name} vs reference output")
    exact = oracle.paged_attention(g["q"], g["k_cache"], g["v_cache"], g["block_tables"], g["seq_lens"],
                                   float(g["scale"]), dt, g["alibi"] if g["alibi"].size else None)
    assert_close(got.float().cpu().numpy(), exact, atol, rtol, f"{name} vs exact oracle")


# ---- the reference's own case list (U(0,1) data, identity tables) ---------------------------------

# reference test/infiniop/paged_attention.py:95-109 and test/infinicore/ops/paged_attention.py:22-37
REFERENCE_CASES = [
    (1, 1, 1, 128, 16, 1024), (4, 40, 40, 128, 16, 1024), (6, 40, 40, 128, 16, 1024), (3, 8, 8, 128, 16, 1024),
    (3, 8, 8, 64, 16, 1024), (8, 64, 8, 128, 16, 2048), (1, 16, 16, 192, 16, 256), (1, 16, 16, 576, 16, 256),
    (1, 16, 1, 576, 16, 256, 512), (1, 24, 4, 256, 16, 32), (1, 12, 2, 256, 16, 32), (1, 6, 1, 256, 16, 32),
    (1, 1, 1, 128, 16, 15),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", REFERENCE_CASES)
def test_reference_case_list(abi, case, dtype):
    num_seqs, heads, kvh, hd, bs, max_len = case[:6]
    vd = case[6] if len(case) > 6 else hd
    g = torch.Generator().manual_seed(sum(case))
    max_blocks = (max_len + bs - 1) // bs
    c = workloads.build_case("ref", dtype=dtype, seq_lens=torch.randint(1, max_len, (num_seqs,), generator=g),
                             num_heads=heads, num_kv_heads=kvh, head_size=hd, value_size=vd, block_size=bs,
                             num_blocks=num_seqs * max_blocks, max_blocks_per_seq=max_blocks, shuffle_tables=False,
                             seed=sum(case))
    # the reference draws U(0,1)
    gg = torch.Generator().manual_seed(sum(case) + 1)
    c.q = torch.rand(c.q.shape, generator=gg).to(dtype)
    c.k_cache = torch.rand(c.k_cache.shape, generator=gg).to(dtype)
    c.v_cache = torch.rand(c.v_cache.shape, generator=gg).to(dtype)
    c.name = f"ref{case}"
    check(c, run_case(abi, c, None), oracle_out(c))


# ---- benchmark configuration 1, as a flow: cache the newest token, then attend ----------------------

@pytest.mark.parametrize("path", PATHS)
def test_config1_caching_then_attention(abi, path):
    c = workloads.config1_small(seed=1)
    d = c.to("cuda")
    abi.paged_caching(d.k_cache, d.v_cache, d.new_k, d.new_v, d.slot_mapping)
    kb, vb = torch_to_bits(c.k_cache).copy(), torch_to_bits(c.v_cache).copy()
    oracle.paged_caching(kb, vb, torch_to_bits(c.new_k), torch_to_bits(c.new_v), c.slot_mapping.numpy())
    assert np.array_equal(torch_to_bits(d.k_cache), kb) and np.array_equal(torch_to_bits(d.v_cache), vb)
    got = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale, path=path)
    want = oracle.paged_attention(torch_to_bits(c.q), kb, vb, c.block_tables.numpy(), c.seq_lens.numpy(), c.scale, 12)
    check(c, got, want)


# ---- edge cases ------------------------------------------------------------------------------------

@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype,heads,kvh,hd", [(torch.float16, 4, 1, 64), (torch.bfloat16, 8, 1, 128), (torch.bfloat16, 2, 2, 128),
                                                (torch.float16, 12, 1, 128), (torch.bfloat16, 20, 2, 64)])
def test_every_length_across_three_pages(abi, path, dtype, heads, kvh, hd):
    """Sequence lengths 1..49 in one batch: every position of the ragged last tile, page boundaries,
    group sizes 1, 4, 8, 10 and 12 (more than one 8-head tile per kv-head)."""
    lens = torch.arange(1, 50)
    c = workloads.build_case("lens1to49", dtype=dtype, seq_lens=lens, num_heads=heads, num_kv_heads=kvh, head_size=hd,
                             block_size=16, seed=21, slack_blocks=7)
    check(c, run_case(abi, c, path), oracle_out(c))


@pytest.mark.parametrize("path", PATHS)
def test_empty_sequences_leave_their_rows_untouched(abi, path):
    c = workloads.build_case("with_empty", dtype=torch.bfloat16, seq_lens=[40, 0, 17, 0, 0, 300], num_heads=8, num_kv_heads=2,
                             head_size=128, block_size=16, seed=22)
    out = torch.full((6, 8, 128), 3.0, dtype=torch.bfloat16, device="cuda")
    got = run_case(abi, c, path, out=out)
    want = oracle_out(c)
    live = [0, 2, 5]
    atol, rtol = ATTN_TOL[c.dtype]
    assert_close(got[live].float().cpu().numpy(), want[live], atol, rtol, "live rows")
    assert bool((got[[1, 3, 4]] == 3.0).all())


def test_all_sequences_empty(abi):
    c = workloads.build_case("all_empty", dtype=torch.float16, seq_lens=[0, 0], num_heads=4, num_kv_heads=2, head_size=64,
                             block_size=16, num_blocks=2, seed=23)
    out = torch.full((2, 4, 64), 5.0, dtype=torch.float16, device="cuda")
    got = run_case(abi, c, None, out=out)
    assert bool((got == 5.0).all())


@pytest.mark.parametrize("path", PATHS)
def test_unused_cache_slots_may_hold_nan(abi, path):
    """Slots past seq_len in the last page, and blocks no table points at, are never part of the
    result even when they hold NaN/Inf bit patterns."""
    c = workloads.build_case("poison", dtype=torch.bfloat16, seq_lens=[5, 33, 47, 16], num_heads=8, num_kv_heads=2, head_size=128,
                             block_size=16, seed=24, slack_blocks=5)
    want = oracle_out(c)
    poison = torch.tensor(float("nan"), dtype=torch.bfloat16)
    used = torch.zeros(c.k_cache.shape[0], dtype=torch.bool)
    for i, ln in enumerate(c.seq_lens.tolist()):
        nblk = (ln + 15) // 16
        used[c.block_tables[i, :nblk]] = True
        if ln % 16:
            last = int(c.block_tables[i, nblk - 1])
            c.k_cache[last, :, ln % 16:, :] = poison
            c.v_cache[last, :, ln % 16:, :] = float("inf")
    c.k_cache[~used] = poison
    c.v_cache[~used] = poison
    got = run_case(abi, c, path)
    assert bool(torch.isfinite(got.float()).all())
    check(c, got, want)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("index_dtype", ["I32", "U32"])
def test_32bit_index_dtypes(abi, path, index_dtype):
    from infinicore_b200.libinfiniop import InfiniDtype

    c = workloads.build_case("idx32", dtype=torch.float16, seq_lens=[100, 3, 64], num_heads=8, num_kv_heads=2, head_size=128,
                             block_size=16, seed=25)
    got = run_case(abi, c, path, index_dtype=getattr(InfiniDtype, index_dtype))
    check(c, got, oracle_out(c))


@pytest.mark.parametrize("path", PATHS)
def test_alibi(abi, path):
    c = workloads.build_case("alibi", dtype=torch.bfloat16, seq_lens=[130, 48, 1], num_heads=8, num_kv_heads=2, head_size=128,
                             block_size=16, seed=26)
    slopes = torch.tensor([2.0 ** (-(i + 1)) for i in range(8)], dtype=torch.float32)
    slopes[3] = 0.0
    check(c, run_case(abi, c, path, alibi=slopes), oracle_out(c, alibi=slopes))


@pytest.mark.parametrize("path", PATHS)
def test_permuted_cache_layout_and_strided_q_out(abi, path):
    """Caches allocated [blocks, slots, heads, dim] and passed as the permuted view (reference
    test/infinicore/ops/paged_caching.py:147-149); q and out are slices of wider buffers."""
    c = workloads.build_case("permuted", dtype=torch.float16, seq_lens=[70, 129, 16], num_heads=8, num_kv_heads=4, head_size=64,
                             block_size=16, seed=27)
    want = oracle_out(c)
    d = c.to("cuda")
    kc = d.k_cache.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    vc = d.v_cache.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert kc.stride() != d.k_cache.stride()
    q_wide = torch.zeros((3, 8, 96), dtype=torch.float16, device="cuda")
    q_wide[:, :, 16:80] = d.q
    out_wide = torch.zeros((3, 16, 64), dtype=torch.float16, device="cuda")
    got = abi.paged_attention(q_wide[:, :, 16:80], kc, vc, d.block_tables, d.seq_lens, d.scale, path=path, out=out_wide[:, ::2])
    check(c, got, want)
    assert bool((out_wide[:, 1::2] == 0).all())


@pytest.mark.parametrize("path", PATHS)
def test_block_size_32_and_wide_block_table(abi, path):
    c = workloads.build_case("bs32", dtype=torch.bfloat16, seq_lens=[200, 31, 97], num_heads=4, num_kv_heads=2, head_size=128,
                             block_size=32, max_blocks_per_seq=40, seed=28)
    check(c, run_case(abi, c, path), oracle_out(c))


@pytest.mark.parametrize("path", ["stream-plan-kernel", "stream-3x4", "stream-combine", "stream-pool", "stream-pool-combine", "stream-row-boxes"])
def test_stream_path_variants(abi, path):
    """The separate plan kernel with plain (non-programmatic) launches, another ring geometry, the combine
    kernel in place of the merge inside the main kernel, one copy per tensor and tile instead of one per
    column chunk, and the chunk pool (ranges too short here to be
    cut: the pool variants must behave like the plain ones), on ragged lengths with empty sequences and a
    split long sequence."""
    c = workloads.build_case("variants", dtype=torch.bfloat16, seq_lens=[1, 0, 47, 5000, 16, 333, 0, 2049], num_heads=32, num_kv_heads=8,
                             head_size=128, block_size=16, seed=33)
    out = torch.full((8, 32, 128), 2.0, dtype=torch.bfloat16, device="cuda")
    got = run_case(abi, c, path, out=out)
    want = oracle_out(c)
    live = [0, 2, 3, 4, 5, 7]
    atol, rtol = ATTN_TOL[c.dtype]
    assert_close(got[live].float().cpu().numpy(), want[live], atol, rtol, path)
    assert bool((got[[1, 6]] == 2.0).all())


@pytest.mark.parametrize("path", ["stream", "stream-combine", "stream-pool", "stream-pool-combine"])
@pytest.mark.parametrize("shape", ["few_long_units", "many_units"])
def test_pieces_and_merges_match_the_oracle_and_repeat_bit_for_bit(abi, path, shape):
    """Ranges long enough to be cut into a head piece and pool chunks (when the pool is on): every way of
    merging the split units - inside the main kernel by the last worker to arrive, or by the combine
    kernel - against the oracle, and three runs bit-identical (piece boundaries and merge order are fixed
    by the plan; which worker computes a chunk is not)."""
    g = torch.Generator().manual_seed(35)
    if shape == "few_long_units":
        # 12 sequences x 8 kv-heads = 96 units of 600..1300 tiles over 1184 workers: a unit collects many records
        lens = torch.randint(9000, 21000, (12,), generator=g)
        lens[3] = 33
        lens[7] = 1
        kw = dict(num_heads=32, num_kv_heads=8)
    else:
        # 700 sequences x 2 kv-heads = 1400 units, more than workers: most units whole, the rest cut once or twice
        lens = torch.randint(300, 1500, (700,), generator=g)
        lens[5] = 0
        kw = dict(num_heads=8, num_kv_heads=2)
    c = workloads.build_case("pieces_" + shape, dtype=torch.bfloat16, seq_lens=lens, head_size=128, block_size=16, seed=35, **kw)
    want = oracle_out(c)
    live = (lens > 0).nonzero().flatten().tolist()
    atol, rtol = ATTN_TOL[c.dtype]
    d = c.to("cuda")
    runs = []
    for _ in range(3):
        out = torch.full((len(lens), kw["num_heads"], 128), 3.0, dtype=torch.bfloat16, device="cuda")
        runs.append(abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale, path=path, out=out).clone())
    assert_close(runs[0][live].float().cpu().numpy(), want[live], atol, rtol, f"{shape} {path}")
    for r in runs[1:]:
        assert torch.equal(r.view(torch.int16), runs[0].view(torch.int16)), "runs differ"
    if shape == "many_units":
        assert bool((runs[0][5] == 3.0).all())


def test_more_sequences_than_the_embedded_plan_holds(abi):
    """5000 short sequences: beyond 4095 the plan comes from the separate plan kernel."""
    g = torch.Generator().manual_seed(34)
    lens = torch.randint(0, 40, (5000,), generator=g)
    c = workloads.build_case("many", dtype=torch.float16, seq_lens=lens, num_heads=4, num_kv_heads=1, head_size=64,
                             block_size=16, seed=34, max_blocks_per_seq=3)
    out = torch.full((5000, 4, 64), 6.0, dtype=torch.float16, device="cuda")
    got = run_case(abi, c, "stream", out=out)
    want = oracle_out(c)
    live = (lens > 0).nonzero().flatten().tolist()
    dead = (lens == 0).nonzero().flatten().tolist()
    atol, rtol = ATTN_TOL[c.dtype]
    assert_close(got[live].float().cpu().numpy(), want[live], atol, rtol, "5000 sequences")
    assert bool((got[dead] == 6.0).all())


def test_block_size_8_takes_the_generic_path(abi):
    c = workloads.build_case("bs8", dtype=torch.float16, seq_lens=[50, 9], num_heads=4, num_kv_heads=2, head_size=64,
                             block_size=8, seed=29)
    check(c, run_case(abi, c, None), oracle_out(c))


# ---- scaled-down versions of the ragged and long-context benchmark configurations ------------------

def test_ragged_lengths_log_uniform(abi):
    """Shape of benchmark configuration 3 (64/8 heads, N(0, 0.5), log-uniform lengths) at 1/16 scale."""
    g = torch.Generator().manual_seed(30)
    u = torch.rand(48, generator=g)
    lens = torch.exp(math.log(16) + u * (math.log(2048) - math.log(16))).round().long()
    c = workloads.build_case("ragged", dtype=torch.bfloat16, seq_lens=lens, num_heads=64, num_kv_heads=8, head_size=128,
                             block_size=16, max_blocks_per_seq=128, std=0.5, seed=30, slack_blocks=16)
    check(c, run_case(abi, c, None), oracle_out(c))


def test_long_context_small_batch_is_split_many_ways(abi):
    """Shape of benchmark configuration 4 (fp16, 2 sequences, 32/8 heads) at 16384 tokens: each
    (sequence, kv-head) is spread over dozens of workers and reduced by the combine kernel."""
    c = workloads.build_case("longctx", dtype=torch.float16, seq_lens=[16384, 16384], num_heads=32, num_kv_heads=8, head_size=128,
                             block_size=16, seed=31)
    check(c, run_case(abi, c, None), oracle_out(c))


# ---- size-independent properties at the full size of benchmark configuration 2 -----------------------

@pytest.fixture(scope="module")
def config2():
    return workloads.config2_llama8b(device="cuda")


def test_config2_subset_against_oracle(abi, config2):
    """Full-size launch (64 x 4096 tokens, 1 GiB of KV); three of the 64 sequences are checked
    element-wise against the oracle."""
    d = config2
    got = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale)
    pick = [0, 31, 63]
    want = oracle.paged_attention(torch_to_bits(d.q[pick]), torch_to_bits(d.k_cache), torch_to_bits(d.v_cache),
                                  d.block_tables[pick].cpu().numpy(), d.seq_lens[pick].cpu().numpy(), d.scale, 19)
    atol, rtol = ATTN_TOL[torch.bfloat16]
    assert_close(got[pick].float().cpu().numpy(), want, atol, rtol, "config 2 subset")
    assert bool(torch.isfinite(got.float()).all())


def test_config2_is_invariant_under_physical_block_permutation(abi, config2):
    """Moving every page to a different physical block (and rewriting the tables to match) must not
    change a single output bit: the result depends on logical content only."""
    d = config2
    base = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale)
    nb = d.k_cache.shape[0]
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(99)).cuda()  # new_pool[perm[b]] = old_pool[b]
    k2 = torch.empty_like(d.k_cache)
    v2 = torch.empty_like(d.v_cache)
    k2[perm] = d.k_cache
    v2[perm] = d.v_cache
    got = abi.paged_attention(d.q, k2, v2, perm[d.block_tables], d.seq_lens, d.scale)
    assert torch.equal(got.view(torch.int16), base.view(torch.int16))


def test_config2_output_is_linear_in_v(abi, config2):
    """Doubling V doubles the output exactly (power-of-two scaling commutes with every rounding)."""
    d = config2
    base = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale)
    got = abi.paged_attention(d.q, d.k_cache, d.v_cache * 2, d.block_tables, d.seq_lens, d.scale)
    assert torch.equal(got.view(torch.int16), (base * 2).view(torch.int16))


def test_config2_repeated_calls_are_deterministic(abi, config2):
    d = config2
    a = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale)
    b = abi.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.scale)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


# ---- ABI behaviour -----------------------------------------------------------------------------------

def _small(dtype=torch.float16, hd=128):
    return workloads.build_case("abi", dtype=dtype, seq_lens=[20, 5], num_heads=4, num_kv_heads=2, head_size=hd,
                                block_size=16, seed=40).to("cuda")


def test_descriptor_validation_status_codes(abi):
    d = _small()
    out = torch.zeros_like(d.q)

    def status(**kw):
        args = dict(out=out, q=d.q, k_cache=d.k_cache, v_cache=d.v_cache, block_tables=d.block_tables,
                    seq_lens=d.seq_lens, alibi=None, scale=d.scale)
        args.update(kw)
        op = abi.AttentionOp(**args)
        st = op.status
        op.destroy()
        return st

    assert status() == 0
    assert status(q=d.q.float()) == 10                                   # F32 is not a decode dtype
    assert status(k_cache=d.k_cache.to(torch.bfloat16)) == 10           # cache dtype must match q
    assert status(seq_lens=d.seq_lens.to(torch.int32)) == 10            # index dtypes must agree
    assert status(block_tables=d.block_tables.float()) == 10
    assert status(q=d.q[0]) == 11                                        # rank
    assert status(block_tables=d.block_tables[0]) == 11
    assert status(out=out[:, :2]) == 11                                  # out heads != q heads
    assert status(q=d.q[:, :3], out=out[:, :3]) == 11                    # 3 q-heads over 2 kv-heads
    assert status(q=d.q[:, :, :96], out=out[:, :, :96], k_cache=d.k_cache[..., :96], v_cache=d.v_cache[..., :96]) == 11  # head size 96
    assert status(q=d.q.transpose(1, 2).contiguous().transpose(1, 2)) == 12  # last dim not dense
    assert status(alibi=torch.zeros(4, dtype=torch.float16, device="cuda")) == 10
    assert status(seq_lens=d.seq_lens[:1]) == 11


def test_insufficient_workspace_is_reported_before_any_launch(abi):
    d = _small()
    out = torch.full_like(d.q, 9.0)
    op = abi.AttentionOp(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale)
    assert op.status == 0 and op.workspace_size > 0
    assert op.run(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, workspace_size=op.workspace_size - 1) == 13
    torch.cuda.synchronize()
    assert bool((out == 9.0).all())
    assert op.run(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens) == 0
    torch.cuda.synchronize()
    op.destroy()


def test_descriptor_reports_its_device(abi):
    import ctypes

    from infinicore_b200.libinfiniop import LIBINFINIOP

    d = _small()
    op = abi.AttentionOp(torch.zeros_like(d.q), d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale)
    dev, idx = ctypes.c_int(-1), ctypes.c_int(-1)
    assert LIBINFINIOP.infiniopGetDescriptorDeviceType(op.desc, ctypes.byref(dev)) == 0 and dev.value == 1
    assert LIBINFINIOP.infiniopGetDescriptorDeviceId(op.desc, ctypes.byref(idx)) == 0 and idx.value == 0
    assert op.desc.contents.device == 1 and op.desc.contents.device_id == 0  # the two leading ints callers read
    op.destroy()


def test_one_descriptor_serves_new_pointers_and_new_lengths(abi):
    """The descriptor holds shapes and strides only; data pointers, lengths and tables are per call."""
    c1 = workloads.build_case("a", dtype=torch.bfloat16, seq_lens=[100, 7, 64], num_heads=8, num_kv_heads=2, head_size=128,
                              block_size=16, num_blocks=32, max_blocks_per_seq=8, seed=41)
    c2 = workloads.build_case("b", dtype=torch.bfloat16, seq_lens=[1, 128, 33], num_heads=8, num_kv_heads=2, head_size=128,
                              block_size=16, num_blocks=32, max_blocks_per_seq=8, seed=42)
    d1, d2 = c1.to("cuda"), c2.to("cuda")
    out = torch.zeros_like(d1.q)
    op = abi.AttentionOp(out, d1.q, d1.k_cache, d1.v_cache, d1.block_tables, d1.seq_lens, None, d1.scale)
    for c, d in ((c1, d1), (c2, d2), (c1, d1)):
        assert op.run(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens) == 0
        torch.cuda.synchronize()
        check(c, out, oracle_out(c))
    op.destroy()


def test_cuda_graph_capture_of_the_decode_step(abi):
    """caching + attention captured into a CUDA graph through the infinirt API and replayed after the
    inputs changed in place (execute allocates nothing and never synchronises)."""
    import ctypes

    from infinicore_b200.libinfiniop import LIBINFINIOP, check_error

    c = workloads.build_case("graph", dtype=torch.bfloat16, seq_lens=[100, 37, 64, 5], num_heads=8, num_kv_heads=2, head_size=128,
                             block_size=16, seed=43)
    d = c.to("cuda")
    out = torch.zeros_like(d.q)
    op = abi.AttentionOp(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale)
    st, cdesc = abi.create_caching(d.k_cache, d.v_cache, d.new_k, d.new_v, d.slot_mapping)
    assert st == 0 and op.status == 0

    stream = ctypes.c_void_p()
    check_error(LIBINFINIOP.infinirtStreamCreate(ctypes.byref(stream)))

    def step(s):
        check_error(LIBINFINIOP.infiniopPagedCaching(cdesc, None, 0, d.k_cache.data_ptr(), d.v_cache.data_ptr(),
                                                     d.new_k.data_ptr(), d.new_v.data_ptr(), d.slot_mapping.data_ptr(), s))
        check_error(op.run(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, stream=s))

    step(stream)  # warm-up outside capture
    check_error(LIBINFINIOP.infinirtStreamSynchronize(stream))
    torch.cuda.synchronize()
    check_error(LIBINFINIOP.infinirtStreamBeginCapture(stream, 2))  # RELAXED, as infinicore's graph does
    step(stream)
    graph = ctypes.c_void_p()
    check_error(LIBINFINIOP.infinirtStreamEndCapture(stream, ctypes.byref(graph)))
    gexec = ctypes.c_void_p()
    check_error(LIBINFINIOP.infinirtGraphInstantiate(ctypes.byref(gexec), graph, None, None, 0))

    # change the inputs in place, replay, compare with the oracle on the new inputs
    g = torch.Generator().manual_seed(44)
    c.q = torch.randn(c.q.shape, generator=g).to(torch.bfloat16)
    c.new_k = torch.randn(c.new_k.shape, generator=g).to(torch.bfloat16)
    c.new_v = torch.randn(c.new_v.shape, generator=g).to(torch.bfloat16)
    d.q.copy_(c.q)
    d.new_k.copy_(c.new_k)
    d.new_v.copy_(c.new_v)
    out.zero_()
    torch.cuda.synchronize()
    check_error(LIBINFINIOP.infinirtGraphLuanch(gexec, stream))
    check_error(LIBINFINIOP.infinirtStreamSynchronize(stream))

    kb, vb = torch_to_bits(c.k_cache).copy(), torch_to_bits(c.v_cache).copy()
    oracle.paged_caching(kb, vb, torch_to_bits(c.new_k), torch_to_bits(c.new_v), c.slot_mapping.numpy())
    want = oracle.paged_attention(torch_to_bits(c.q), kb, vb, c.block_tables.numpy(), c.seq_lens.numpy(), c.scale, 19)
    check(c, out, want)
    assert np.array_equal(torch_to_bits(d.k_cache), kb)

    check_error(LIBINFINIOP.infinirtGraphExecDestroy(gexec))
    check_error(LIBINFINIOP.infinirtGraphDestroy(graph))
    check_error(LIBINFINIOP.infinirtStreamDestroy(stream))
    check_error(LIBINFINIOP.infiniopDestroyPagedCachingDescriptor(cdesc))
    op.destroy()


def test_python_operators_match_the_abi_path(abi):
    """infinicore_b200.paged_attention / paged_caching (descriptor cache, torch's current stream)."""
    import infinicore_b200 as ib

    c = workloads.config1_small(seed=3)
    d = c.to("cuda")
    ib.paged_caching(d.k_cache, d.v_cache, d.new_k, d.new_v, d.slot_mapping)
    got = ib.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale)
    again = ib.paged_attention(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale)
    torch.cuda.synchronize()
    kb, vb = torch_to_bits(c.k_cache).copy(), torch_to_bits(c.v_cache).copy()
    oracle.paged_caching(kb, vb, torch_to_bits(c.new_k), torch_to_bits(c.new_v), c.slot_mapping.numpy())
    want = oracle.paged_attention(torch_to_bits(c.q), kb, vb, c.block_tables.numpy(), c.seq_lens.numpy(), c.scale, 12)
    check(c, got, want)
    assert torch.equal(got, again)


@pytest.mark.parametrize("direct_output", [False, True, "auto"])
def test_decode_step_graph_replay_matches_direct_calls(abi, direct_output):
    """infinicore_b200.DecodeStep: host inputs -> H2D -> caching -> attention -> D2H captured once and
    replayed; two replays with different inputs, each checked against the oracle.  With direct_output the
    kernels store the rows into the pinned host buffer themselves (no copy node)."""
    import infinicore_b200 as ib

    base = workloads.build_case("step", dtype=torch.bfloat16, seq_lens=[100, 37, 64, 5, 900, 16], num_heads=32, num_kv_heads=8,
                                head_size=128, block_size=16, seed=61)
    d = base.to("cuda")
    step = ib.DecodeStep(d.k_cache, d.v_cache, num_seqs=6, num_heads=32, max_blocks_per_seq=base.block_tables.shape[1],
                         scale=base.scale, direct_output=direct_output)
    kb, vb = torch_to_bits(base.k_cache).copy(), torch_to_bits(base.v_cache).copy()
    g = torch.Generator().manual_seed(62)
    for round_ in range(2):
        q = torch.randn(base.q.shape, generator=g).to(torch.bfloat16)
        nk = torch.randn(base.new_k.shape, generator=g).to(torch.bfloat16)
        nv = torch.randn(base.new_v.shape, generator=g).to(torch.bfloat16)
        step.host["q"].copy_(q)
        step.host["new_k"].copy_(nk)
        step.host["new_v"].copy_(nv)
        step.host["slot_mapping"].copy_(base.slot_mapping)
        step.host["block_tables"].copy_(base.block_tables)
        step.host["seq_lens"].copy_(base.seq_lens)
        got = step.run().clone()
        oracle.paged_caching(kb, vb, torch_to_bits(nk), torch_to_bits(nv), base.slot_mapping.numpy())
        want = oracle.paged_attention(torch_to_bits(q), kb, vb, base.block_tables.numpy(), base.seq_lens.numpy(), base.scale, 19)
        check(base, got, want)
        assert np.array_equal(torch_to_bits(d.k_cache), kb), f"round {round_}: pools differ"


# ---- key width 576: the four-warp wide-head kernel (and the generic kernel beside it) -------------------

WIDE_PATHS = [None, "generic", "stream-3x4", "stream-chunk-boxes"]


@pytest.mark.parametrize("path", WIDE_PATHS)
@pytest.mark.parametrize("dtype,heads,kvh,value,bs", [(torch.bfloat16, 16, 1, 512, 16), (torch.float16, 8, 2, 576, 16),
                                                      (torch.bfloat16, 24, 2, 576, 32), (torch.float16, 128, 1, 512, 64),
                                                      (torch.bfloat16, 3, 1, 576, 16)])
def test_wide_heads_every_length_across_pages(abi, path, dtype, heads, kvh, value, bs):
    """Lengths 1..2*block+2 plus a few long ones and an empty one: every ragged last tile, page and tile
    boundaries; latent attention (values 512 wide) and plain 576; 1, 2, 3 and 16 eight-head tiles per
    kv-head, one of them partly filled; many more ranges than units, so units are split and combined."""
    lens = list(range(1, 2 * bs + 3)) + [0, 700, 1025, 333]
    c = workloads.build_case("wide", dtype=dtype, seq_lens=lens, num_heads=heads, num_kv_heads=kvh, head_size=576, value_size=value,
                             block_size=bs, seed=61, std=0.3, slack_blocks=5)
    check(c, run_case(abi, c, path), oracle_out(c))


@pytest.mark.parametrize("path", WIDE_PATHS)
def test_wide_heads_alibi_int32_and_poisoned_slots(abi, path):
    from infinicore_b200.libinfiniop import InfiniDtype

    c = workloads.build_case("wide_alibi", dtype=torch.bfloat16, seq_lens=[130, 48, 1, 2000, 17], num_heads=16, num_kv_heads=2,
                             head_size=576, value_size=512, block_size=16, seed=62, std=0.3, slack_blocks=4)
    slopes = -torch.linspace(0.0, 0.2, 16, dtype=torch.float32)
    want = oracle_out(c, alibi=slopes)
    poison = torch.tensor(float("nan"), dtype=torch.bfloat16)
    used = torch.zeros(c.k_cache.shape[0], dtype=torch.bool)
    for i, ln in enumerate(c.seq_lens.tolist()):
        nblk = (ln + 15) // 16
        used[c.block_tables[i, :nblk]] = True
        if ln % 16:
            last = int(c.block_tables[i, nblk - 1])
            c.k_cache[last, :, ln % 16:, :] = poison
            c.v_cache[last, :, ln % 16:, :] = float("inf")
    c.k_cache[~used] = poison
    c.v_cache[~used] = poison
    got = run_case(abi, c, path, alibi=slopes, index_dtype=InfiniDtype.I32)
    assert bool(torch.isfinite(got.float()).all())
    check(c, got, want)


def test_wide_heads_long_batch_matches_generic_kernel(abi):
    """64 x 1500 tokens of latent attention with 32 heads: streaming result against the row-wise kernel's."""
    c = workloads.build_case("wide_long", dtype=torch.bfloat16, seq_lens=[1500 + 7 * i for i in range(64)], num_heads=32, num_kv_heads=1,
                             head_size=576, value_size=512, block_size=16, seed=63, std=0.3)
    a = run_case(abi, c, None)
    b = run_case(abi, c, "generic")
    atol, rtol = ATTN_TOL[c.dtype]
    assert_close(a.float().cpu().numpy(), b.float().cpu().numpy(), atol, rtol, "wide vs generic")


@pytest.mark.parametrize("dtype,heads,value,hd,bs", [(torch.bfloat16, 128, 512, 576, 16), (torch.float16, 16, 576, 576, 32),
                                                    (torch.bfloat16, 32, 128, 128, 16), (torch.float16, 8, 64, 64, 16)])
def test_copies_per_chunk_and_per_tensor_give_the_same_bits(abi, dtype, heads, value, hd, bs):
    """The two ways of fetching a tile (one copy per 64-element column chunk through the 4-D tensor maps, one per
    tensor through the 5-D maps) move the same bytes to the same places: bit-identical outputs, at key width 576
    (where the 5-D maps are the default) and at head 128 / 64 (where they are not)."""
    c = workloads.build_case("boxes", dtype=dtype, seq_lens=[2500, 31, 700, 1, 4097, 16], num_heads=heads, num_kv_heads=1 if hd == 576 else 4,
                             head_size=hd, value_size=value, block_size=bs, seed=66, std=0.3)
    a = run_case(abi, c, "stream-chunk-boxes")
    b = run_case(abi, c, "stream-row-boxes")
    assert np.array_equal(torch_to_bits(a), torch_to_bits(b))
    check(c, b, oracle_out(c))


# ---- several destinations for the output rows (what the KV-head-sharded mode stores into its peers) -------

@pytest.mark.parametrize("path", [None, "generic", "stream-3x4"])
@pytest.mark.parametrize("dtype,heads,kvh,hd,value", [(torch.bfloat16, 8, 2, 128, 128), (torch.float16, 12, 1, 64, 64),
                                                      (torch.bfloat16, 16, 1, 576, 512)])
def test_multi_out_stores_every_destination(abi, path, dtype, heads, kvh, hd, value):
    """Three destinations, each the same head slice of a wider buffer (as a rank's slice inside every
    rank's full output): all equal the single-output result, nothing outside the slices is touched,
    rows of empty sequences stay untouched everywhere.  Long and short sequences, so that both the
    direct stores of the main kernels and the combine kernel's stores are exercised."""
    import infinicore_b200 as ib

    lens = [3000, 17, 0, 260, 1, 1500]
    c = workloads.build_case("multi", dtype=dtype, seq_lens=lens, num_heads=heads, num_kv_heads=kvh, head_size=hd, value_size=value,
                             block_size=16, seed=71, std=0.4).to("cuda")
    single = run_case(abi, c, path)
    wide = [torch.full((len(lens), 3 * heads, value), 9.0, dtype=dtype, device="cuda") for _ in range(3)]
    outs = [w[:, heads:2 * heads] for w in wide]
    if path is None:
        # through the Python operator (tensors and a raw address mixed)
        ib.paged_attention_multi_out([outs[0], outs[1], outs[2].data_ptr()], c.q, c.k_cache, c.v_cache, c.block_tables, c.seq_lens,
                                     None, c.scale)
    else:
        # through the C ABI with a descriptor created under this path's environment
        import ctypes

        from infinicore_b200.libinfiniop import LIBINFINIOP, check_error

        op = abi.AttentionOp(outs[0], c.q, c.k_cache, c.v_cache, c.block_tables, c.seq_lens, None, c.scale, path)
        check_error(op.status)
        try:
            arr = (ctypes.c_void_p * 3)(*[o.data_ptr() for o in outs])
            check_error(LIBINFINIOP.infiniopPagedAttentionMultiOut(
                op.desc, op.workspace.data(), op.workspace_size, arr, 3, c.q.data_ptr(), c.k_cache.data_ptr(), c.v_cache.data_ptr(),
                c.block_tables.data_ptr(), c.seq_lens.data_ptr(), None, None))
            torch.cuda.synchronize()
        finally:
            op.destroy()
    torch.cuda.synchronize()
    live = [i for i, n in enumerate(lens) if n > 0]
    for w, o in zip(wide, outs):
        assert torch.equal(o[live], single[live])
        assert bool((o[2] == 9.0).all())                                       # the empty sequence's row
        assert bool((w[:, :heads] == 9.0).all()) and bool((w[:, 2 * heads:] == 9.0).all())  # outside the slice
    check(c, outs[0][live].contiguous(), oracle_out(c.to("cpu"))[live])


def test_multi_out_argument_checks(abi):
    import ctypes

    from infinicore_b200.libinfiniop import LIBINFINIOP

    c = workloads.build_case("multi_bad", dtype=torch.float16, seq_lens=[5, 6], num_heads=4, num_kv_heads=2, head_size=64, block_size=16,
                             seed=72).to("cuda")
    out = torch.zeros_like(c.q)
    op = abi.AttentionOp(out, c.q, c.k_cache, c.v_cache, c.block_tables, c.seq_lens, None, c.scale)
    try:
        args = (c.q.data_ptr(), c.k_cache.data_ptr(), c.v_cache.data_ptr(), c.block_tables.data_ptr(), c.seq_lens.data_ptr(), None, None)
        one = (ctypes.c_void_p * 1)(out.data_ptr())
        nine = (ctypes.c_void_p * 9)(*([out.data_ptr()] * 9))
        hole = (ctypes.c_void_p * 2)(out.data_ptr(), None)
        assert LIBINFINIOP.infiniopPagedAttentionMultiOut(op.desc, op.workspace.data(), op.workspace_size, None, 1, *args) == 4
        assert LIBINFINIOP.infiniopPagedAttentionMultiOut(op.desc, op.workspace.data(), op.workspace_size, one, 0, *args) == 3
        assert LIBINFINIOP.infiniopPagedAttentionMultiOut(op.desc, op.workspace.data(), op.workspace_size, nine, 9, *args) == 3
        assert LIBINFINIOP.infiniopPagedAttentionMultiOut(op.desc, op.workspace.data(), op.workspace_size, hole, 2, *args) == 4
        assert LIBINFINIOP.infiniopPagedAttentionMultiOut(op.desc, op.workspace.data(), op.workspace_size, one, 1, *args) == 0
        torch.cuda.synchronize()
    finally:
        op.destroy()
