"""GPU parity of infiniopRoPE through the C ABI, bit for bit.

The oracle restates the reference's CPU kernel (src/infiniop/ops/rope/cpu/rope_cpu.cc:34-105) and is
pinned against the reference's own torch checker by the golden files; the CUDA kernel computes in the
same order with the same roundings, so every comparison here is exact (the reference's test allows
fp16 1e-3 / 1e-2, bf16 5e-3 / 5e-2, fp32 1e-4 / 1e-3: test/infiniop/rope.py:46-50).  Shapes and strides
are the reference test's (test/infiniop/rope.py:27-38), out of place and in place, both pairings."""
import numpy as np
import pytest
import torch

import oracle
from helpers import bits_to_torch, golden_names, load_golden, torch_to_bits
from infinicore_b200.libinfiniop import InfiniDtype

pytestmark = pytest.mark.gpu

CODE = {torch.float16: 12, torch.bfloat16: 19, torch.float32: 13, torch.float64: 14}
GPT_J, GPT_NEOX = 0, 1


@pytest.fixture(scope="module")
def abi():
    import abi as _abi

    yield _abi


def strided(shape, strides, dtype, gen):
    if strides is None:
        return torch.randn(shape, generator=gen).to(dtype)
    extent = 1 + sum((n - 1) * s for n, s in zip(shape, strides))
    return torch.randn(extent, generator=gen).to(dtype).as_strided(shape, strides)


def tables(table_len, dhead, dtype, theta=1e5):
    freqs = 1.0 / (theta ** (torch.arange(0, dhead, 2)[: dhead // 2].float() / dhead))
    angles = torch.outer(torch.arange(table_len).float(), freqs)
    return torch.sin(angles).to(dtype), torch.cos(angles).to(dtype)


def to_cuda_like(t):
    """Device copy with the same strides (storage extent included)."""
    if t.is_contiguous():
        return t.cuda()
    extent = 1 + sum((n - 1) * s for n, s in zip(t.shape, t.stride()))
    base = torch.zeros(extent, dtype=t.dtype, device="cuda")
    view = base.as_strided(t.shape, t.stride())
    view.copy_(t.cuda())
    return view


def as_bits(t):
    """numpy view of a CPU tensor that keeps its strides (uint16 patterns for 16-bit types)."""
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def check(abi, x, pos, sin, cos, algo, y_strides=None, inplace=False, pos_dtype=None):
    dt = CODE[x.dtype]
    want = oracle.rope(as_bits(x), pos.numpy(), as_bits(sin), as_bits(cos), dt, algo == GPT_J)
    xd = to_cuda_like(x)
    if inplace:
        yd = xd
    elif y_strides is None:
        yd = torch.zeros(x.shape, dtype=x.dtype, device="cuda")
    else:
        yd = to_cuda_like(strided(x.shape, y_strides, x.dtype, torch.Generator().manual_seed(5)))
    pd = pos.cuda() if pos_dtype is None else pos.to(pos_dtype[0]).cuda()
    got = abi.rope(xd, pd, sin.cuda(), cos.cuda(), algo, y=yd, pos_dtype=pos_dtype[1] if pos_dtype else None)
    assert np.array_equal(torch_to_bits(got), want), "differs from the oracle"
    if not inplace:
        assert torch.equal(xd.cpu(), x), "x was modified"


@pytest.mark.parametrize("name", golden_names("rope_"))
def test_golden(abi, name):
    g = load_golden(name)
    dt = int(g["dtype"])
    x = bits_to_torch(g["x"], dt)
    if g["x_strides"].size:
        extent = 1 + sum((n - 1) * int(s) for n, s in zip(x.shape, g["x_strides"]))
        base = torch.zeros(extent, dtype=x.dtype)
        view = base.as_strided(x.shape, [int(s) for s in g["x_strides"]])
        view.copy_(x)
        x = view
    got = abi.rope(to_cuda_like(x), torch.from_numpy(g["pos_ids"]).cuda(), bits_to_torch(g["sin_table"], dt).cuda(),
                   bits_to_torch(g["cos_table"], dt).cuda(), int(g["algo"]))
    assert np.array_equal(torch_to_bits(got), g["y"])


# (shape, x_strides, y_strides): reference test/infiniop/rope.py:27-38
REFERENCE_CASES = [
    ((1, 32, 128), None, None),
    ((10, 32, 64), None, None),
    ((4, 1, 32), (64, 64, 1), None),
    ((11, 33, 128), None, (8000, 200, 1)),
    ((3, 32, 128), (8000, 200, 1), (7000, 128, 1)),
    ((8, 1, 32, 128), None, None),
    ((8, 10, 32, 64), None, None),
    ((8, 20, 32, 64), (40960, 64, 1280, 1), (40960, 64, 1280, 1)),
    ((8, 20, 4, 64), (1048576, 64, 262144, 1), (1048576, 64, 262144, 1)),
]


@pytest.mark.parametrize("algo", [GPT_J, GPT_NEOX])
@pytest.mark.parametrize("inplace", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape,x_strides,y_strides", REFERENCE_CASES)
def test_reference_cases(abi, shape, x_strides, y_strides, dtype, inplace, algo):
    if inplace and x_strides != y_strides:
        pytest.skip("in place needs equal strides (as in the reference test)")
    gen = torch.Generator().manual_seed(hash((shape, algo)) & 0xffff)
    x = strided(shape, x_strides, dtype, gen)
    seqlen, dhead = shape[-3], shape[-1]
    pos = torch.arange(seqlen, dtype=torch.int64)  # the reference test's positions
    sin, cos = tables(seqlen, dhead, dtype)
    check(abi, x, pos, sin, cos, algo, y_strides, inplace, pos_dtype=(torch.int32, InfiniDtype.I32))


@pytest.mark.parametrize("torch_dtype,code", [(torch.int8, InfiniDtype.I8), (torch.uint8, InfiniDtype.U8), (torch.int16, InfiniDtype.I16),
                                             (torch.int32, InfiniDtype.I32), (torch.int64, InfiniDtype.I64),
                                             (torch.uint16, InfiniDtype.U16), (torch.uint32, InfiniDtype.U32), (torch.uint64, InfiniDtype.U64)])
def test_every_position_type(abi, torch_dtype, code):
    gen = torch.Generator().manual_seed(3)
    x = torch.randn((9, 4, 64), generator=gen).to(torch.bfloat16)
    pos = torch.randint(0, 100, (9,), generator=gen)
    sin, cos = tables(100, 64, torch.bfloat16)
    check(abi, x, pos, sin, cos, GPT_NEOX, pos_dtype=(torch_dtype, code))


def test_per_batch_positions_and_float64(abi):
    gen = torch.Generator().manual_seed(4)
    x = torch.randn((3, 6, 2, 32), generator=gen, dtype=torch.float64)
    pos = torch.randint(0, 50, (3, 6), generator=gen)
    sin, cos = tables(50, 32, torch.float64)
    check(abi, x, pos, sin, cos, GPT_J)
    check(abi, x, pos, sin, cos, GPT_NEOX)


def test_positions_outside_the_tables_copy_their_rows(abi):
    gen = torch.Generator().manual_seed(6)
    x = torch.randn((5, 3, 64), generator=gen).to(torch.float16)
    pos = torch.tensor([2, -1, 7, 8, 0], dtype=torch.int64)  # table_len 8: -1 and 8 are outside
    sin, cos = tables(8, 64, torch.float16)
    check(abi, x, pos, sin, cos, GPT_NEOX)
    got = abi.rope(x.cuda(), pos.cuda(), sin.cuda(), cos.cuda(), GPT_J)
    assert torch.equal(got[1].cpu(), x[1]) and torch.equal(got[3].cpu(), x[3])


def test_partial_rotary_view(abi):
    """Rotating the last 64 of 576 columns (the MLA key layout) is a strided view of the same call."""
    gen = torch.Generator().manual_seed(7)
    full = torch.randn((6, 1, 576), generator=gen).to(torch.bfloat16)
    pos = torch.randint(0, 32, (6,), generator=gen)
    sin, cos = tables(32, 64, torch.bfloat16)
    fd = full.cuda()
    view = fd[:, :, 512:]
    abi.rope(view, pos.cuda(), sin.cuda(), cos.cuda(), GPT_J, y=view)
    want = full.clone()
    rotated = oracle.rope(as_bits(full[:, :, 512:]), pos.numpy(), as_bits(sin), as_bits(cos), 19, True)
    assert np.array_equal(torch_to_bits(fd[:, :, 512:]), rotated)
    assert torch.equal(fd[:, :, :512].cpu(), want[:, :, :512]), "columns outside the view changed"


def test_large_rows_match_the_oracle(abi):
    """A prefill-sized call (2048 tokens x 32 heads x 128): the vector path at scale."""
    gen = torch.Generator().manual_seed(8)
    x = torch.randn((2048, 32, 128), generator=gen).to(torch.bfloat16)
    pos = torch.arange(2048)
    sin, cos = tables(2048, 128, torch.bfloat16)
    check(abi, x, pos, sin, cos, GPT_NEOX)
    check(abi, x, pos, sin, cos, GPT_J, inplace=True)


@pytest.mark.parametrize("algo", [GPT_J, GPT_NEOX])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prefill_sized_calls(abi, dtype, algo):
    """Calls of a thousand tokens and more on the vector path: an odd token count, a batch dimension with
    per-batch positions, strided rows (q as a slice of a fused qkv buffer), 8 and 40 heads, positions outside
    the tables, in place."""
    gen = torch.Generator().manual_seed(9)
    sin, cos = tables(300, 128, dtype)
    # 1025 tokens x 8 heads: the second token of the last pair does not exist
    x = torch.randn((1025, 8, 128), generator=gen).to(dtype)
    pos = torch.randint(0, 300, (1025,), generator=gen)
    pos[7] = 300  # outside: the row is copied
    pos[1024] = -1
    check(abi, x, pos, sin, cos, algo)
    # batch 3 x 400 tokens x 40 heads, positions per batch, rows strided (a head is 128 of 192 columns), in place
    x4 = strided((3, 400, 40, 128), (400 * 40 * 192, 40 * 192, 192, 1), dtype, gen)
    pos4 = torch.randint(0, 300, (3, 400), generator=gen)
    check(abi, x4, pos4, sin, cos, algo, inplace=True)
    # head 64 (4 or 8 items per row), separate strided output
    sin64, cos64 = tables(300, 64, dtype)
    x64 = torch.randn((1500, 16, 64), generator=gen).to(dtype)
    check(abi, x64, torch.randint(0, 300, (1500,), generator=gen), sin64, cos64, algo, y_strides=(16 * 80, 80, 1))


def test_rejected_inputs(abi):
    x = torch.zeros((4, 2, 64), dtype=torch.float16, device="cuda")
    pos = torch.zeros(4, dtype=torch.int64, device="cuda")
    sin = torch.zeros((8, 32), dtype=torch.float16, device="cuda")
    bad = lambda *a, **k: abi.rope_create(*a, **k)[0]
    assert bad(x, x, pos, sin, sin.to(torch.bfloat16), GPT_J) == 10          # table dtype differs
    assert bad(x, x, pos.float(), sin, sin, GPT_J) == 10                     # positions must be integers
    assert bad(x, x[:3], pos, sin, sin, GPT_J) == 11                         # x / y shapes differ
    assert bad(x, x, pos[:3], sin, sin, GPT_J) == 11                         # one position per token
    assert bad(x, x, pos, sin[:, :16], sin[:, :16], GPT_J) == 11             # dhead != 2 * table_dim
    assert bad(x, x, pos, sin.t().contiguous().t(), sin, GPT_J) == 12        # tables must be contiguous
    assert bad(x, x.transpose(1, 2).contiguous().transpose(1, 2), pos, sin, sin, GPT_J) == 12  # last stride 1
    assert bad(x, x, pos, sin, sin, 2) == 4                                  # algorithm outside the enum (the reference's status)
    assert bad(x.int(), x.int(), pos, sin.int(), sin.int(), GPT_J) == 10     # data type
