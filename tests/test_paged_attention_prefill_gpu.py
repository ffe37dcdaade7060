"""GPU parity of infiniopPagedAttentionPrefill through the C ABI: against the reference checker's
golden outputs and the CPU oracle ("exact" mode) on the same seeded inputs, on both kernels - the
tensor-core tile kernel (default where eligible) and the row-wise generic kernel
(INFINIOP_PAGED_PREFILL_PATH=generic at descriptor creation).  Tolerance: the decode path's
(fp16 atol 2e-3 / rtol 2e-3, bf16 atol 1e-2 / rtol 1e-2), tighter than the reference's own prefill
test (fp16 1e-2, bf16 2e-2; test/infiniop/paged_attention_prefill.py:45-48)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import ATTN_TOL, assert_close, bits_to_float, bits_to_torch, golden_names, load_golden, torch_to_bits
from infinicore_b200 import workloads

pytestmark = pytest.mark.gpu

PATHS = [None, "generic", "tiles"]
PATHS_HD128 = [None, "generic", "tiles", "umma", "umma-q1", "umma-q2-s3"]  # the tcgen05 kernel takes head sizes 64 and 128 (and is the default there)


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def oracle_out(c, alibi=None):
    dt = 12 if c.dtype == torch.float16 else 19
    return oracle.paged_attention_prefill(
        torch_to_bits(c.q), torch_to_bits(c.k_cache), torch_to_bits(c.v_cache), c.block_tables.cpu().numpy(),
        c.seq_lens.cpu().numpy(), c.cum_seq_lens_q.cpu().numpy(), c.scale, dt,
        alibi.cpu().numpy() if alibi is not None else None)


def run_case(abi, c, path, alibi=None, index_dtype=None, out=None):
    d = c.to("cuda")
    return abi.paged_attention_prefill(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.cum_seq_lens_q, d.scale,
                                       alibi.cuda() if alibi is not None else None, path=path, out=out, index_dtype=index_dtype)


def check(c, got, want):
    atol, rtol = ATTN_TOL[c.dtype]
    assert_close(got.float().cpu().numpy(), want, atol, rtol, c.name)


@pytest.mark.parametrize("path", PATHS_HD128)
@pytest.mark.parametrize("name", golden_names("prefill_"))
def test_golden(abi, name, path):
    if path is not None and path.startswith("umma") and "hd128" not in name and "hd64" not in name:
        pytest.skip("tcgen05 kernel: head sizes 64 and 128 only")
    if path == "tiles" and "576" in name:
        pytest.skip("tile kernel: head sizes 64 and 128")
    g = load_golden(name)
    dt = int(g["dtype"])
    q, kc, vc = (bits_to_torch(g[k], dt).cuda() for k in ("q", "k_cache", "v_cache"))
    got = abi.paged_attention_prefill(q, kc, vc, torch.from_numpy(g["block_tables"]).cuda(), torch.from_numpy(g["seq_lens"]).cuda(),
                                      torch.from_numpy(g["cum_seq_lens_q"]).cuda(), float(g["scale"]), path=path)
    atol, rtol = ATTN_TOL[dt]
    assert_close(got.float().cpu().numpy(), bits_to_float(g["out"], dt), atol, rtol, f"{name} vs reference output")


# reference test/infiniop/paged_attention_prefill.py:25-44:
# (num_seqs, heads, kv_heads, head, block, max_step_len, rounds, index dtype[, value])
REFERENCE_CASES = [
    (1, 1, 1, 128, 8, 16, 1), (1, 4, 4, 128, 8, 16, 4), (2, 8, 8, 128, 16, 32, 2), (4, 16, 16, 128, 8, 64, 3),
    (8, 64, 64, 128, 8, 16, 5), (16, 128, 128, 128, 8, 16, 4), (2, 16, 1, 576, 16, 8, 2, 512),
]


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", REFERENCE_CASES)
def test_reference_case_list_multi_round(abi, case, dtype, index_dtype):
    """The reference test's flow: several rounds, each appending a random number of new tokens per
    sequence to a growing cache, prefill attention over cache + new tokens each round."""
    num_seqs, heads, kvh, hd, bs, max_step, rounds = case[:7]
    vd = case[7] if len(case) > 7 else hd
    g = torch.Generator().manual_seed(sum(case))
    cached = torch.zeros(num_seqs, dtype=torch.int64)
    for r in range(rounds):
        new = torch.randint(1, max_step + 1, (num_seqs,), generator=g)
        c = workloads.build_prefill_case(f"ref{case}r{r}", dtype=dtype, new_lens=new, cached_lens=cached, num_heads=heads,
                                         num_kv_heads=kvh, head_size=hd, value_size=vd, block_size=bs, seed=sum(case) + r,
                                         index_dtype=index_dtype, std=0.5 if hd == 576 else 1.0)
        from infinicore_b200.libinfiniop import InfiniDtype

        idt = InfiniDtype.I32 if index_dtype == torch.int32 else None
        check(c, run_case(abi, c, None, index_dtype=idt), oracle_out(c))
        cached = cached + new


@pytest.mark.parametrize("path", PATHS_HD128)
@pytest.mark.parametrize("dtype,heads,kvh,hd,bs", [(torch.bfloat16, 8, 2, 128, 16), (torch.float16, 4, 1, 64, 16),
                                                   (torch.bfloat16, 4, 4, 128, 8), (torch.float16, 8, 2, 128, 32)])
def test_gqa_ragged_chunks_and_tile_boundaries(abi, path, dtype, heads, kvh, hd, bs):
    if path is not None and path.startswith("umma") and hd not in (64, 128):
        pytest.skip("tcgen05 kernel: head sizes 64 and 128 only")
    """Chunk lengths around the 64-row tile and the page size, cached prefixes of every alignment,
    one sequence with no new tokens."""
    new = [1, 63, 64, 65, 127, 128, 129, 0, 200, 17]
    cached = [0, 1, 15, 16, 64, 0, 130, 50, 3, 999]
    c = workloads.build_prefill_case("ragged", dtype=dtype, new_lens=new, cached_lens=cached, num_heads=heads, num_kv_heads=kvh,
                                     head_size=hd, block_size=bs, seed=91)
    check(c, run_case(abi, c, path), oracle_out(c))


@pytest.mark.parametrize("path", PATHS_HD128)
def test_alibi(abi, path):
    c = workloads.build_prefill_case("alibi", dtype=torch.bfloat16, new_lens=[70, 9], cached_lens=[30, 0], num_heads=8,
                                     num_kv_heads=2, head_size=128, block_size=16, seed=92)
    slopes = torch.tensor([2.0 ** (-(i + 1)) for i in range(8)], dtype=torch.float32)
    slopes[5] = 0.0
    check(c, run_case(abi, c, path, alibi=slopes), oracle_out(c, alibi=slopes))


@pytest.mark.parametrize("path", PATHS_HD128)
def test_unused_cache_slots_may_hold_nan_and_untouched_rows_stay(abi, path):
    c = workloads.build_prefill_case("poison", dtype=torch.float16, new_lens=[37, 80], cached_lens=[5, 0], num_heads=4,
                                     num_kv_heads=2, head_size=128, block_size=16, seed=93)
    want = oracle_out(c)
    used = torch.zeros(c.k_cache.shape[0], dtype=torch.bool)
    for i, ln in enumerate(c.seq_lens.tolist()):
        nblk = (ln + 15) // 16
        used[c.block_tables[i, :nblk]] = True
        if ln % 16:
            last = int(c.block_tables[i, nblk - 1])
            c.k_cache[last, :, ln % 16:, :] = float("nan")
            c.v_cache[last, :, ln % 16:, :] = float("inf")
    c.k_cache[~used] = float("nan")
    c.v_cache[~used] = float("nan")
    # q/out carry 3 extra rows that no chunk covers: they must not be written
    d = c.to("cuda")
    q_big = torch.cat([d.q, torch.zeros((3, 4, 128), dtype=torch.float16, device="cuda")])
    out_big = torch.full((q_big.shape[0], 4, 128), 8.0, dtype=torch.float16, device="cuda")
    got = abi.paged_attention_prefill(q_big, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.cum_seq_lens_q, d.scale,
                                      path=path, out=out_big)
    assert bool(torch.isfinite(got.float()).all())
    check(c, got[:-3], want)
    assert bool((got[-3:] == 8.0).all())


@pytest.mark.parametrize("path", ["tiles", "umma", "umma-q1", "umma-q2-s3"])
def test_long_prompt_against_oracle(abi, path):
    """2 prompts x 1024 new tokens over 512 cached, Llama-3-8B head shape."""
    c = workloads.build_prefill_case("long", dtype=torch.bfloat16, new_lens=[1024, 1000], cached_lens=[512, 0], num_heads=32,
                                     num_kv_heads=8, head_size=128, block_size=16, seed=94)
    check(c, run_case(abi, c, path), oracle_out(c))


@pytest.mark.parametrize("path", ["umma-late-v", "umma-late-v-k2"])
def test_late_value_tiles_change_nothing(abi, path):
    """V copies held back (a test switch of the producers): the softmax warps store P of two tiles while the P.V
    issuer still waits for the first one's values.  Every barrier the issuer can fall behind on exists once per
    score buffer, so it reads their phases rightly: same bits as the undisturbed run, nothing reported."""
    c = workloads.build_prefill_case("late_v", dtype=torch.bfloat16, new_lens=[700, 129], cached_lens=[300, 0], num_heads=8,
                                     num_kv_heads=2, head_size=128, block_size=16, seed=97)
    want = run_case(abi, c, "umma")
    got = run_case(abi, c, path)
    assert torch.equal(got.cpu(), want.cpu())
    assert abi.kernel_status() == 0
    check(c, got, oracle_out(c))


def test_prefill_of_one_token_equals_decode(abi):
    """A chunk of one new token per sequence is the decode problem: same result as infiniopPagedAttention
    within rounding of the two kernels."""
    dc = workloads.build_case("eq", dtype=torch.bfloat16, seq_lens=[100, 37, 64, 5, 900], num_heads=32, num_kv_heads=8,
                              head_size=128, block_size=16, seed=95).to("cuda")
    dec = abi.paged_attention(dc.q, dc.k_cache, dc.v_cache, dc.block_tables, dc.seq_lens, dc.scale)
    cum = torch.arange(6, dtype=torch.int64, device="cuda")
    pre = abi.paged_attention_prefill(dc.q, dc.k_cache, dc.v_cache, dc.block_tables, dc.seq_lens, cum, dc.scale)
    atol, rtol = ATTN_TOL[torch.bfloat16]
    assert_close(pre.float().cpu().numpy(), dec.float().cpu().numpy(), atol, rtol, "prefill(1 token) vs decode")


def test_descriptor_validation_status_codes(abi):
    c = workloads.build_prefill_case("abi", dtype=torch.float16, new_lens=[5, 9], cached_lens=[3, 0], num_heads=4, num_kv_heads=2,
                                     head_size=128, block_size=16, seed=96).to("cuda")
    out = torch.zeros_like(c.q)

    def status(**kw):
        args = dict(out=out, q=c.q, k_cache=c.k_cache, v_cache=c.v_cache, block_tables=c.block_tables, seq_lens=c.seq_lens,
                    cum_q=c.cum_seq_lens_q, alibi=None, scale=c.scale)
        args.update(kw)
        st, desc = abi.create_prefill(**args)
        if st == 0:
            from infinicore_b200.libinfiniop import LIBINFINIOP

            LIBINFINIOP.infiniopDestroyPagedAttentionPrefillDescriptor(desc)
        return st

    assert status() == 0
    assert status(q=c.q.float()) == 10
    assert status(seq_lens=c.seq_lens.to(torch.int32)) == 10            # index dtypes must agree
    assert status(cum_q=c.cum_seq_lens_q[:-1]) == 3                     # BAD_PARAM: needs num_seqs + 1 entries
    assert status(q=c.q[0]) == 11
    assert status(out=out[:, :2]) == 11
    assert status(q=c.q[:, :3], out=out[:, :3]) == 11                   # 3 q-heads over 2 kv-heads
    assert status(q=c.q.transpose(1, 2).contiguous().transpose(1, 2)) == 12


def test_python_operator(abi):
    import infinicore_b200 as ib

    c = workloads.build_prefill_case("py", dtype=torch.bfloat16, new_lens=[70, 33], cached_lens=[10, 0], num_heads=8, num_kv_heads=2,
                                     head_size=128, block_size=16, seed=97)
    d = c.to("cuda")
    got = ib.paged_attention_prefill(d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.cum_seq_lens_q, None, d.scale)
    torch.cuda.synchronize()
    check(c, got, oracle_out(c))
