"""GPU parity of infiniopKVCaching through the C ABI, bit for bit (the reference's own test demands
atol = rtol = 0: test/infiniop/kv_caching.py:62-66).  Cache shapes and strides are the reference test's
(test/infiniop/kv_caching.py:48-56), including its non-unit last stride and its padded layouts."""
import numpy as np
import pytest
import torch

import oracle
from helpers import bits_to_torch, golden_names, load_golden, torch_to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def strided(shape, strides, dtype, gen):
    if strides is None:
        return torch.randn(shape, generator=gen).to(dtype)
    extent = 1 + sum((n - 1) * s for n, s in zip(shape, strides))
    return torch.randn(extent, generator=gen).to(dtype).as_strided(shape, strides)


def to_cuda_like(t):
    """Device copy with the same strides; returns (view, whole storage) so that gaps can be checked too."""
    extent = 1 + sum((n - 1) * s for n, s in zip(t.shape, t.stride()))
    base = torch.zeros(extent, dtype=t.dtype, device="cuda")
    view = base.as_strided(t.shape, t.stride())
    view.copy_(t.cuda())
    return view, base


def np_view(t):
    """numpy view of a CPU tensor that keeps its strides (raw bit patterns for 16-bit types)."""
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def check(abi, k_cache, v_cache, k, v, past, len_dtype=torch.int64):
    kd, k_base = to_cuda_like(k_cache)
    vd, v_base = to_cuda_like(v_cache)
    nk, _ = to_cuda_like(k)
    nv, _ = to_cuda_like(v)
    k_before, v_before = k_base.clone(), v_base.clone()
    abi.kv_caching(kd, vd, nk, nv, past.to(len_dtype).cuda())
    want_k, want_v = k_cache.clone(), v_cache.clone()
    oracle.kv_caching(np_view(want_k), np_view(want_v), np_view(k), np_view(v), past.numpy())
    assert np.array_equal(torch_to_bits(kd), torch_to_bits(want_k)), "k_cache differs from the oracle"
    assert np.array_equal(torch_to_bits(vd), torch_to_bits(want_v)), "v_cache differs from the oracle"
    # nothing between the strided rows was touched
    kd.zero_(), vd.zero_()
    k_before.as_strided(k_cache.shape, k_cache.stride()).zero_()
    v_before.as_strided(v_cache.shape, v_cache.stride()).zero_()
    assert torch.equal(k_base, k_before) and torch.equal(v_base, v_before), "bytes outside the cache view changed"


@pytest.mark.parametrize("name", golden_names("kvc_"))
def test_golden(abi, name):
    g = load_golden(name)
    dt = int(g["dtype"])
    dense_k, dense_v = bits_to_torch(g["k_cache"], dt), bits_to_torch(g["v_cache"], dt)
    strides = [int(s) for s in g["cache_strides"]] or None
    gen = torch.Generator().manual_seed(0)
    kc, vc = strided(dense_k.shape, strides, dense_k.dtype, gen), strided(dense_k.shape, strides, dense_k.dtype, gen)
    kc.copy_(dense_k), vc.copy_(dense_v)
    kd, _ = to_cuda_like(kc)
    vd, _ = to_cuda_like(vc)
    abi.kv_caching(kd, vd, bits_to_torch(g["k"], dt).cuda(), bits_to_torch(g["v"], dt).cuda(), torch.from_numpy(g["past_kv_lengths"]).cuda())
    assert np.array_equal(torch_to_bits(kd), g["k_cache_after"])
    assert np.array_equal(torch_to_bits(vd), g["v_cache_after"])


# (cache shape, cache strides): reference test/infiniop/kv_caching.py:48-56
REFERENCE_CASES = [
    ((1, 1, 8, 1), None),
    ((1, 8, 32, 32), None),
    ((8, 8, 64, 32), None),
    ((1, 32, 8, 64), (32768, 1024, 64, 1)),
    ((4, 8, 32, 16), (65536, 8192, 256, 16)),
    ((8, 16, 64, 128), (8388608, 524288, 8192, 1)),
    ((1, 2, 2304, 128), (589824, 294912, 128, 1)),
]


@pytest.mark.parametrize("len_dtype", [torch.int64, torch.int32])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,strides", REFERENCE_CASES)
def test_reference_cases(abi, shape, strides, dtype, len_dtype):
    gen = torch.Generator().manual_seed(shape[2] * 131 + shape[3])
    seq_len = int(torch.randint(1, shape[2], (1,), generator=gen))
    k_cache, v_cache = strided(shape, strides, dtype, gen), strided(shape, strides, dtype, gen)
    new_shape = (shape[0], shape[1], seq_len, shape[3])
    k, v = torch.randn(new_shape, generator=gen).to(dtype), torch.randn(new_shape, generator=gen).to(dtype)
    past = torch.randint(0, shape[2] - seq_len + 1, (shape[0],), generator=gen)
    check(abi, k_cache, v_cache, k, v, past, len_dtype)


def test_strided_new_rows_and_rows_outside_the_cache(abi):
    """k / v as permuted views ([batch, seq, heads, hidden] storage, the layout a projection produces) and
    lengths that push some rows past the end or before the start of the cache: those rows are skipped."""
    gen = torch.Generator().manual_seed(9)
    k_cache, v_cache = torch.randn((3, 4, 16, 64), generator=gen).bfloat16(), torch.randn((3, 4, 16, 64), generator=gen).bfloat16()
    k = torch.randn((3, 5, 4, 64), generator=gen).bfloat16().permute(0, 2, 1, 3)
    v = torch.randn((3, 5, 4, 64), generator=gen).bfloat16().permute(0, 2, 1, 3)
    check(abi, k_cache, v_cache, k, v, torch.tensor([11, 14, -2]))


def test_decode_sized_append_matches_the_oracle(abi):
    """One new row for each of 64 sequences of an 8-head, 4096-row cache (the contiguous twin of the paged
    decode workload)."""
    gen = torch.Generator().manual_seed(10)
    k_cache = torch.randn((64, 8, 512, 128), generator=gen).bfloat16()
    v_cache = torch.randn((64, 8, 512, 128), generator=gen).bfloat16()
    k, v = torch.randn((64, 8, 1, 128), generator=gen).bfloat16(), torch.randn((64, 8, 1, 128), generator=gen).bfloat16()
    check(abi, k_cache, v_cache, k, v, torch.randint(0, 512, (64,), generator=gen))


def test_python_operator(abi):
    import infinicore_b200 as ib

    gen = torch.Generator().manual_seed(11)
    k_cache, v_cache = torch.randn((2, 2, 8, 32), generator=gen).half(), torch.randn((2, 2, 8, 32), generator=gen).half()
    k, v = torch.randn((2, 2, 3, 32), generator=gen).half(), torch.randn((2, 2, 3, 32), generator=gen).half()
    past = torch.tensor([0, 5])
    kd, vd = k_cache.cuda(), v_cache.cuda()
    ib.kv_caching(kd, vd, k.cuda(), v.cuda(), past.cuda())
    ib.kv_caching(kd, vd, k.cuda(), v.cuda(), past.cuda())  # second call: cached descriptor
    torch.cuda.synchronize()
    oracle.kv_caching(np_view(k_cache), np_view(v_cache), np_view(k), np_view(v), past.numpy())
    assert torch.equal(kd.cpu(), k_cache) and torch.equal(vd.cpu(), v_cache)


def test_rejected_inputs(abi):
    kc = torch.zeros((2, 2, 8, 32), dtype=torch.float16, device="cuda")
    k = torch.zeros((2, 2, 3, 32), dtype=torch.float16, device="cuda")
    past = torch.zeros(2, dtype=torch.int64, device="cuda")
    bad = lambda *a: abi.kv_caching_create(*a)[0]
    assert bad(kc, kc, k, k, past) == 0
    assert bad(kc, kc.float(), k, k, past) == 10                       # cache dtypes differ
    assert bad(kc.double(), kc.double(), k.double(), k.double(), past) == 10   # F64 is not accepted
    assert bad(kc, kc, k, k, past.to(torch.int16)) == 10               # lengths I32 | I64
    assert bad(kc, kc, k[0], k[0], past) == 11                         # rank
    assert bad(kc, kc[:, :, :4], k, k, past) == 11                     # caches of different shape
    assert bad(kc, kc, k, k[:, :, :2], past) == 11                     # new rows of different shape
    assert bad(kc, kc, k[:, :1], k[:, :1], past) == 11                 # head count differs from the cache
    assert bad(kc, kc, k, k, past[:1]) == 11                           # one length per sequence
