"""GPU parity of infiniopPagedCaching through the C ABI: bit-exact against the reference's
golden outputs and against the CPU oracle, whole pool compared (untouched slots included)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import TORCH_DTYPE, bits_to_torch, golden_names, load_golden, torch_to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def _bits(t):
    return torch_to_bits(t)


@pytest.mark.parametrize("name", golden_names("cache_"))
def test_golden_bit_exact(abi, name):
    g = load_golden(name)
    dt = int(g["dtype"])
    dev = "cuda"
    k_phys = bits_to_torch(g["k_cache"], dt).to(dev)
    v_phys = bits_to_torch(g["v_cache"], dt).to(dev)
    k_view, v_view = (k_phys.permute(0, 2, 1, 3), v_phys.permute(0, 2, 1, 3)) if int(g["permuted"]) else (k_phys, v_phys)
    k = bits_to_torch(g["k"], dt).to(dev)
    v = bits_to_torch(g["v"], dt).to(dev)
    slots = torch.from_numpy(g["slot_mapping"]).to(dev)
    abi.paged_caching(k_view, v_view, k, v, slots)
    assert np.array_equal(_bits(k_phys), g["k_cache_after"])
    assert np.array_equal(_bits(v_phys), g["v_cache_after"])


# reference test/infiniop/paged_caching.py:61-73: (num_seqs, max_seq_len, kv_heads, head, block[, value])
REFERENCE_CASES = [
    (1, 128, 8, 128, 16), (5, 512, 40, 128, 16), (16, 1024, 8, 64, 32), (10, 1024, 40, 64, 32), (2, 128, 1, 576, 16, 512),
]


@pytest.mark.parametrize("case", REFERENCE_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_reference_case_list_against_oracle(abi, case, dtype):
    num_seqs, max_len, kvh, hd, bs = case[:5]
    vd = case[5] if len(case) > 5 else hd
    num_blocks = 512
    g = torch.Generator().manual_seed(hash(case) % 1000)
    lens = torch.randint(1, max_len + 1, (num_seqs,), generator=g)
    lens = torch.minimum(lens, torch.tensor(num_blocks * bs // num_seqs))
    ntok = int(lens.sum())
    slots = torch.arange(ntok, dtype=torch.int64)  # contiguous ascending, as the reference test builds it
    k_cache = torch.rand((num_blocks, kvh, bs, hd), generator=g).to(dtype)
    v_cache = torch.rand((num_blocks, kvh, bs, vd), generator=g).to(dtype)
    k = torch.rand((ntok, kvh, hd), generator=g).to(dtype)
    v = torch.rand((ntok, kvh, vd), generator=g).to(dtype)

    want_k, want_v = _bits(k_cache).copy(), _bits(v_cache).copy()
    oracle.paged_caching(want_k, want_v, _bits(k), _bits(v), slots.numpy())

    dk, dv = k_cache.cuda(), v_cache.cuda()
    abi.paged_caching(dk, dv, k.cuda(), v.cuda(), slots.cuda())
    assert np.array_equal(_bits(dk), want_k)
    assert np.array_equal(_bits(dv), want_v)


def test_negative_slots_are_padding_and_untouched_slots_stay_bit_identical(abi):
    g = torch.Generator().manual_seed(5)
    # pools hold arbitrary bit patterns, NaNs included: a byte mover must not care
    k_cache = torch.randint(-32768, 32767, (64, 4, 16, 128), generator=g, dtype=torch.int16).view(torch.bfloat16)
    v_cache = torch.randint(-32768, 32767, (64, 4, 16, 128), generator=g, dtype=torch.int16).view(torch.bfloat16)
    k = torch.randn((33, 4, 128), generator=g).to(torch.bfloat16)
    v = torch.randn((33, 4, 128), generator=g).to(torch.bfloat16)
    slots = torch.randperm(64 * 16, generator=g)[:33].to(torch.int64)
    slots[::4] = -1
    want_k, want_v = _bits(k_cache).copy(), _bits(v_cache).copy()
    oracle.paged_caching(want_k, want_v, _bits(k), _bits(v), slots.numpy())
    dk, dv = k_cache.cuda(), v_cache.cuda()
    abi.paged_caching(dk, dv, k.cuda(), v.cuda(), slots.cuda())
    assert np.array_equal(_bits(dk), want_k) and np.array_equal(_bits(dv), want_v)
    assert (slots < 0).sum() == 9


def test_unaligned_bases_and_strided_sources_take_the_element_path(abi):
    g = torch.Generator().manual_seed(6)
    pool = torch.randn(2 * (8 * 2 * 16 * 64) + 8, generator=g).to(torch.float16).cuda()
    k_cache = pool[1:1 + 8 * 2 * 16 * 64].view(8, 2, 16, 64)       # base 2 bytes off a 16-byte boundary
    v_cache = pool[8 * 2 * 16 * 64 + 3:8 * 2 * 16 * 64 * 2 + 3].view(8, 2, 16, 64)
    src = torch.randn((10, 2, 2, 64), generator=g).to(torch.float16).cuda()
    k, v = src[:, 0], src[:, 1]                                      # token stride 256, head stride 64
    slots = torch.randperm(8 * 16, generator=g)[:10].to(torch.int64)
    want_k, want_v = _bits(k_cache).copy(), _bits(v_cache).copy()
    oracle.paged_caching(want_k, want_v, _bits(k), _bits(v), slots.numpy())
    abi.paged_caching(k_cache, v_cache, k, v, slots.cuda())
    assert np.array_equal(_bits(k_cache), want_k) and np.array_equal(_bits(v_cache), want_v)


def test_multi_round_cache_manager(abi):
    """Rounds of appends with blocks handed out on demand (reference
    test/infiniop/paged_caching_prefill.py): state after every round equals the oracle's."""
    g = torch.Generator().manual_seed(7)
    kvh, hd, bs, nb = 8, 128, 8, 256
    k_cache = torch.zeros((nb, kvh, bs, hd), dtype=torch.float16)
    v_cache = torch.zeros((nb, kvh, bs, hd), dtype=torch.float16)
    dk, dv = k_cache.cuda(), v_cache.cuda()
    ok, ov = _bits(k_cache).copy(), _bits(v_cache).copy()
    free = list(torch.randperm(nb, generator=g).numpy())
    tables = {i: [] for i in range(4)}
    lens = {i: 0 for i in range(4)}
    for _ in range(5):
        slots, rows = [], 0
        for i in range(4):
            add = int(torch.randint(1, 40, (1,), generator=g))
            for _t in range(add):
                if lens[i] % bs == 0:
                    tables[i].append(int(free.pop()))
                slots.append(tables[i][lens[i] // bs] * bs + lens[i] % bs)
                lens[i] += 1
                rows += 1
        k = torch.randn((rows, kvh, hd), generator=g).to(torch.float16)
        v = torch.randn((rows, kvh, hd), generator=g).to(torch.float16)
        sm = torch.tensor(slots, dtype=torch.int64)
        oracle.paged_caching(ok, ov, _bits(k), _bits(v), sm.numpy())
        abi.paged_caching(dk, dv, k.cuda(), v.cuda(), sm.cuda())
        assert np.array_equal(_bits(dk), ok) and np.array_equal(_bits(dv), ov)


def test_descriptor_validation_status_codes(abi):
    dev = "cuda"
    kc = torch.zeros((4, 2, 16, 64), dtype=torch.float16, device=dev)
    k = torch.zeros((3, 2, 64), dtype=torch.float16, device=dev)
    sm = torch.zeros(3, dtype=torch.int64, device=dev)
    assert abi.create_caching(kc, kc, k, k, sm)[0] == 0
    assert abi.create_caching(kc, kc, k, k, sm.to(torch.int32))[0] == 10        # slot_mapping must be I64
    assert abi.create_caching(kc, kc.to(torch.bfloat16), k, k, sm)[0] == 10     # mixed dtypes
    assert abi.create_caching(kc, kc, k[:, :1], k, sm)[0] == 11                 # head count mismatch
    assert abi.create_caching(kc, kc, k[:2], k, sm)[0] == 11                    # token count mismatch
    assert abi.create_caching(kc[0], kc, k, k, sm)[0] == 11                     # cache rank < 4
    assert abi.create_caching(kc, kc, k.to(torch.float64), k, sm)[0] == 10


def test_zero_tokens_is_a_no_op(abi):
    kc = torch.ones((4, 2, 16, 64), dtype=torch.float16, device="cuda")
    k = torch.zeros((0, 2, 64), dtype=torch.float16, device="cuda")
    abi.paged_caching(kc, kc.clone(), k, k, torch.zeros(0, dtype=torch.int64, device="cuda"))
    assert bool((kc == 1).all())
