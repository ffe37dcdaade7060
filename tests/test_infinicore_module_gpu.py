"""The pybind module and its `infinicore`-style facade, driven the way the reference drives its own
(test/infinicore/ops/paged_attention.py, test/infinicore/ops/paged_caching.py): the reference's case lists
(:22-37 and :22-34), its input recipe (uniform random values, identity block tables, random lengths; slots
handed out contiguously; the cache handed in as a permuted view for the [blocks, block, heads, width]
layout), its tolerances, and its two call forms (returning / out=)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close, torch_to_bits

pytestmark = pytest.mark.gpu

# (num_seqs, num_heads, num_kv_heads, head_size, block_size, max_seq_len, use_alibi[, value_size])
ATTENTION_CASES = [
    (1, 1, 1, 128, 16, 15, False),
    (4, 40, 40, 128, 16, 1024, False),
    (6, 40, 40, 128, 16, 1024, False),
    (3, 8, 8, 128, 16, 1024, False),
    (3, 8, 8, 64, 16, 1024, False),
    (8, 64, 8, 128, 16, 2048, False),
    (1, 24, 4, 256, 16, 32, False),
    (1, 12, 2, 256, 16, 32, False),
    (1, 6, 1, 256, 16, 32, False),
    (1, 16, 1, 576, 16, 32, False, 512),
]
ATTENTION_TOLERANCE = {torch.float16: (0.0, 1e-2), torch.bfloat16: (0.0, 5e-2)}

# (num_seqs, max_seq_len, num_kv_heads, head_size, block_size, permute_dim_1_2[, value_size])
CACHING_CASES = [
    (1, 128, 8, 128, 16, False),
    (1, 128, 8, 128, 16, True),
    (5, 512, 40, 256, 16, False),
    (5, 512, 40, 256, 16, True),
    (16, 1024, 8, 64, 32, False),
    (16, 1024, 8, 64, 32, True),
    (10, 1024, 40, 64, 32, False),
    (10, 1024, 40, 64, 32, True),
    (1, 32, 1, 576, 16, False, 512),
]


@pytest.fixture(scope="module")
def infinicore():
    import infinicore_b200.infinicore as m

    return m


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
@pytest.mark.parametrize("case", ATTENTION_CASES, ids=[f"attn{i}" for i in range(len(ATTENTION_CASES))])
def test_paged_attention_cases_of_the_reference(infinicore, case, dtype):
    num_seqs, num_heads, num_kv_heads, head_size, block_size, max_seq_len, _ = case[:7]
    value_size = case[7] if len(case) > 7 else head_size
    g = torch.Generator().manual_seed(100 + num_seqs * 7 + num_heads)
    max_blocks = (max_seq_len + block_size - 1) // block_size
    num_blocks = num_seqs * max_blocks
    lens = torch.randint(1, max_seq_len, (num_seqs,), dtype=torch.int64, generator=g)
    tables = torch.arange(0, num_seqs * max_blocks, dtype=torch.int64).view(num_seqs, max_blocks)
    q = torch.rand((num_seqs, num_heads, head_size), generator=g).to(dtype)
    kc = torch.rand((num_blocks, num_kv_heads, block_size, head_size), generator=g).to(dtype)
    vc = torch.rand((num_blocks, num_kv_heads, block_size, value_size), generator=g).to(dtype)
    scale = 1.0 / (head_size ** 0.5)
    code = 12 if dtype == torch.float16 else 19
    want = oracle.paged_attention(torch_to_bits(q), torch_to_bits(kc), torch_to_bits(vc), tables.numpy(), lens.numpy(), scale, code,
                                  mode="reference")
    dev = [infinicore.from_torch(t.cuda()) for t in (q, kc, vc, tables, lens)]
    atol, rtol = ATTENTION_TOLERANCE[dtype]

    # the returning form allocates its result (value width)
    out = infinicore.paged_attention(*dev, alibi_slopes=None, scale=scale)
    infinicore.sync_stream()
    assert out.shape == [num_seqs, num_heads, value_size]
    # one rounding of the output type on top of the reference's own tolerance (atol = 0 there)
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    assert_close(out.to_torch().float().cpu().numpy(), want, atol, rtol + ulp, "returning form")

    # the out= form writes where it is told, and agrees bit for bit
    target = torch.zeros((num_seqs, num_heads, value_size), dtype=dtype, device="cuda")
    back = infinicore.paged_attention(*dev, None, scale, out=infinicore.from_torch(target))
    infinicore.sync_stream()
    assert back.data_ptr() == target.data_ptr()
    assert torch.equal(target.view(torch.int16), out.to_torch().view(torch.int16))
    assert infinicore.kernel_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32], ids=["f16", "bf16", "f32"])
@pytest.mark.parametrize("case", CACHING_CASES, ids=[f"cache{i}" for i in range(len(CACHING_CASES))])
def test_paged_caching_cases_of_the_reference(infinicore, case, dtype):
    num_seqs, max_seq_len, num_kv_heads, head_size, block_size, permuted = case[:6]
    value_size = case[6] if len(case) > 6 else head_size
    num_blocks = 4096
    g = torch.Generator().manual_seed(200 + num_seqs + head_size)
    lens = torch.randint(1, max_seq_len + 1, (num_seqs,), dtype=torch.int64, generator=g)
    ntok = int(lens.sum())
    slots = torch.arange(ntok, dtype=torch.int64)  # the scheduler hands out contiguous runs of slots
    k = torch.rand((ntok, num_kv_heads, head_size), generator=g).to(dtype).cuda()
    v = torch.rand((ntok, num_kv_heads, value_size), generator=g).to(dtype).cuda()
    if permuted:
        kc = torch.zeros((num_blocks, block_size, num_kv_heads, head_size), dtype=dtype, device="cuda")
        vc = torch.zeros((num_blocks, block_size, num_kv_heads, value_size), dtype=dtype, device="cuda")
    else:
        kc = torch.zeros((num_blocks, num_kv_heads, block_size, head_size), dtype=dtype, device="cuda")
        vc = torch.zeros((num_blocks, num_kv_heads, block_size, value_size), dtype=dtype, device="cuda")
    tk, tv = infinicore.from_torch(kc), infinicore.from_torch(vc)
    if permuted:
        tk, tv = tk.permute([0, 2, 1, 3]), tv.permute([0, 2, 1, 3])
    got = infinicore.paged_caching(tk, tv, infinicore.from_torch(k), infinicore.from_torch(v), infinicore.from_torch(slots.cuda()))
    infinicore.sync_stream()
    assert got[0] is tk and got[1] is tv

    # what the reference's torch loop writes: token i, head h -> [slot // block, (h, slot % block) or (slot % block, h), :]
    want_k, want_v = torch.zeros_like(kc), torch.zeros_like(vc)
    blk, off = slots // block_size, slots % block_size
    if permuted:
        want_k[blk.cuda(), off.cuda()] = k
        want_v[blk.cuda(), off.cuda()] = v
    else:
        want_k[blk.cuda(), :, off.cuda()] = k
        want_v[blk.cuda(), :, off.cuda()] = v
    assert torch.equal(kc, want_k) and torch.equal(vc, want_v), "the scatter must be bit-exact"
    assert infinicore.kernel_status() == 0


def test_views_keep_their_owner_alive_and_refuse_cpu_tensors(infinicore):
    t = torch.arange(24, dtype=torch.float32, device="cuda").view(2, 3, 4)
    x = infinicore.from_torch(t)
    p = x.permute([2, 0, 1])
    del t, x
    assert p.shape == [4, 2, 3] and p.stride() == [1, 12, 4]
    assert torch.equal(p.to_torch().cpu(), torch.arange(24, dtype=torch.float32).view(2, 3, 4).permute(2, 0, 1))
    with pytest.raises(RuntimeError):
        infinicore.from_torch(torch.zeros(3))


def test_a_refused_call_raises_with_its_status(infinicore):
    q = infinicore.from_torch(torch.zeros((2, 8, 128), dtype=torch.float16, device="cuda"))
    kc = infinicore.from_torch(torch.zeros((4, 3, 16, 128), dtype=torch.float16, device="cuda"))  # 8 heads over 3 kv-heads
    bt = infinicore.from_torch(torch.zeros((2, 2), dtype=torch.int64, device="cuda"))
    lens = infinicore.from_torch(torch.ones((2,), dtype=torch.int64, device="cuda"))
    with pytest.raises(RuntimeError, match="infiniStatus_t"):
        infinicore.paged_attention(q, kc, kc, bt, lens, None, 1.0)
