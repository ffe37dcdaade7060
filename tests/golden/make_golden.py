"""Regenerates tests/golden/*.npz by running the REFERENCE's own Python checkers on seeded inputs.

Run in a container that has the reference checkout (it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/InfiniCore [--only=attention|caching|prefill|rope|kv_caching|layer]

The two functions executed are imported unmodified from the reference tree:
  ref_single_query_cached_kv_attention   test/infiniop/paged_attention.py:47-88
  ref_paged_caching                      test/infiniop/paged_caching.py:25-55
  ref_paged_attention_multi_turn         test/infiniop/paged_attention_prefill.py:96-140
  rotary_embedding, sin_cos_table        test/infiniop/rope.py:87-133 (run with its CPU device value, i.e. fp32 arithmetic)
  torch_kv_caching                       test/infiniop/kv_caching.py:25-41
Those files import the reference's ctypes harness at module level (which would try to load the
reference's compiled library); a stand-in `libinfiniop` module with empty attributes is put
in sys.modules first so that only the pure-torch functions are used.

Each .npz stores the inputs as raw bit patterns (uint16 for fp16/bf16) plus the reference's
output, so the tests need neither torch-specific pickles nor the reference.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from infinicore_b200 import workloads  # noqa: E402


def load_reference(ref_root: Path):
    class _Anything(types.ModuleType):
        def __getattr__(self, name):
            if name.startswith("__"):
                raise AttributeError(name)
            return type(name, (), {"__getattr__": lambda self, n: 0})()

    sys.modules["libinfiniop"] = _Anything("libinfiniop")
    mods = {}
    for name in ("paged_attention", "paged_caching", "paged_attention_prefill", "rope", "kv_caching"):
        spec = importlib.util.spec_from_file_location(f"_ref_{name}", ref_root / "test" / "infiniop" / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods["paged_attention"], mods["paged_caching"], mods["paged_attention_prefill"], mods["rope"], mods["kv_caching"]


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    return t.contiguous().numpy().copy()


DTYPE_CODE = {torch.float16: 12, torch.float32: 13, torch.bfloat16: 19}


def attention_cases():
    g = torch.Generator()
    g.manual_seed(1234)
    yield "attn_c1_fp16_gqa4_hd64", workloads.config1_small(seed=1), None
    yield "attn_bf16_gqa4_hd128", workloads.build_case(
        "x", dtype=torch.bfloat16, seq_lens=[300, 17, 1, 160], num_heads=8, num_kv_heads=2, head_size=128,
        block_size=16, num_blocks=40, seed=11), None
    yield "attn_bf16_gqa8_hd128", workloads.build_case(
        "x", dtype=torch.bfloat16, seq_lens=[64, 333, 16, 15], num_heads=16, num_kv_heads=2, head_size=128,
        block_size=16, num_blocks=32, seed=12, std=0.5), None
    yield "attn_fp16_mha_hd128_alibi", workloads.build_case(
        "x", dtype=torch.float16, seq_lens=[200, 31], num_heads=4, num_kv_heads=4, head_size=128,
        block_size=16, num_blocks=16, seed=13), "alibi"
    yield "attn_fp16_gqa6_hd256", workloads.build_case(
        "x", dtype=torch.float16, seq_lens=[32, 9], num_heads=12, num_kv_heads=2, head_size=256,
        block_size=16, num_blocks=4, seed=14), None
    yield "attn_bf16_mla_hd576_v512", workloads.build_case(
        "x", dtype=torch.bfloat16, seq_lens=[100, 7], num_heads=16, num_kv_heads=1, head_size=576, value_size=512,
        block_size=16, num_blocks=8, seed=15, std=0.3), None
    yield "attn_fp16_gqa2_hd64_bs32", workloads.build_case(
        "x", dtype=torch.float16, seq_lens=[150, 64, 33], num_heads=4, num_kv_heads=2, head_size=64,
        block_size=32, num_blocks=10, seed=16), None
    yield "attn_bf16_mha_hd192", workloads.build_case(
        "x", dtype=torch.bfloat16, seq_lens=[77], num_heads=3, num_kv_heads=3, head_size=192,
        block_size=16, num_blocks=6, seed=17), None


def make_attention(ref_attn):
    for name, case, variant in attention_cases():
        alibi = None
        if variant == "alibi":
            alibi = torch.tensor(ref_attn.get_alibi_slopes(case.num_heads), dtype=torch.float32)
        out = ref_attn.ref_single_query_cached_kv_attention(
            case.q, case.k_cache, case.v_cache, case.block_tables, case.seq_lens, case.scale, alibi)
        np.savez_compressed(
            HERE / f"{name}.npz",
            dtype=np.int64(DTYPE_CODE[case.dtype]), scale=np.float32(case.scale),
            q=bits(case.q), k_cache=bits(case.k_cache), v_cache=bits(case.v_cache),
            block_tables=case.block_tables.numpy(), seq_lens=case.seq_lens.numpy(),
            alibi=(alibi.numpy() if alibi is not None else np.zeros(0, np.float32)),
            out=bits(out),
        )
        print("wrote", name, tuple(out.shape))


def caching_cases():
    # (name, dtype, num_blocks, kv_heads, block_size, head, v_head, num_tokens, permuted layout)
    yield "cache_fp16_hd64", torch.float16, 32, 2, 16, 64, 64, 37, False
    yield "cache_bf16_hd128_bs32", torch.bfloat16, 12, 4, 32, 128, 128, 50, False
    yield "cache_f32_hd64", torch.float32, 16, 2, 16, 64, 64, 21, False
    yield "cache_bf16_mla_576_512", torch.bfloat16, 8, 1, 16, 576, 512, 19, False
    yield "cache_fp16_permuted_layout", torch.float16, 16, 4, 16, 64, 64, 40, True


def make_caching(ref_cache):
    for idx, (name, dtype, nb, kvh, bs, hd, vd, ntok, permuted) in enumerate(caching_cases()):
        g = torch.Generator()
        g.manual_seed(100 + idx)
        if permuted:
            # allocated [nb, bs, kvh, hd], handed over as the [nb, kvh, bs, hd] view
            # (reference test/infinicore/ops/paged_caching.py:147-149)
            k_cache = torch.randn((nb, bs, kvh, hd), generator=g).to(dtype).permute(0, 2, 1, 3)
            v_cache = torch.randn((nb, bs, kvh, vd), generator=g).to(dtype).permute(0, 2, 1, 3)
        else:
            k_cache = torch.randn((nb, kvh, bs, hd), generator=g).to(dtype)
            v_cache = torch.randn((nb, kvh, bs, vd), generator=g).to(dtype)
        k = torch.randn((ntok, kvh, hd), generator=g).to(dtype)
        v = torch.randn((ntok, kvh, vd), generator=g).to(dtype)
        slots = torch.randperm(nb * bs, generator=g)[:ntok].to(torch.int64)
        k_after, v_after = ref_cache.ref_paged_caching(k_cache, v_cache, k, v, slots)
        # pools are stored in their PHYSICAL order; `permuted` tells the test how to view them
        phys = (lambda t: t.permute(0, 2, 1, 3)) if permuted else (lambda t: t)
        np.savez_compressed(
            HERE / f"{name}.npz",
            dtype=np.int64(DTYPE_CODE[dtype]), permuted=np.int64(permuted),
            k_cache=bits(phys(k_cache)), v_cache=bits(phys(v_cache)), k=bits(k), v=bits(v),
            slot_mapping=slots.numpy(),
            k_cache_after=bits(phys(k_after)), v_cache_after=bits(phys(v_after)),
        )
        print("wrote", name)


def prefill_cases():
    # (name, dtype, new_lens, cached_lens, heads, kv_heads, head, block, value)
    # The reference's checker has no repeat_interleave: it covers MHA (and kv_heads == 1, which
    # broadcasts), as do the reference's own prefill test cases.
    yield "prefill_bf16_mha_hd128", torch.bfloat16, [70, 5, 130], [0, 33, 64], 4, 4, 128, 16, None
    yield "prefill_fp16_mha_hd128_bs8", torch.float16, [16, 9, 64, 1], [0, 7, 30, 100], 4, 4, 128, 8, None
    yield "prefill_fp16_mha_hd64", torch.float16, [100, 65], [28, 0], 3, 3, 64, 16, None
    yield "prefill_bf16_mqa_hd128", torch.bfloat16, [40, 17], [9, 0], 8, 1, 128, 16, None
    yield "prefill_bf16_mla_576_512", torch.bfloat16, [8, 3], [0, 8], 16, 1, 576, 16, 512


def make_prefill(ref_prefill):
    for idx, (name, dtype, new, cached, heads, kvh, hd, bs, vd) in enumerate(prefill_cases()):
        c = workloads.build_prefill_case(name, dtype=dtype, new_lens=new, cached_lens=cached, num_heads=heads,
                                         num_kv_heads=kvh, head_size=hd, block_size=bs, seed=200 + idx, value_size=vd,
                                         std=0.5 if hd == 576 else 1.0)
        out = ref_prefill.ref_paged_attention_multi_turn(c.q, c.k_cache, c.v_cache, c.block_tables, c.seq_lens,
                                                         c.cum_seq_lens_q, c.scale)
        np.savez_compressed(
            HERE / f"{name}.npz",
            dtype=np.int64(DTYPE_CODE[dtype]), scale=np.float32(c.scale),
            q=bits(c.q), k_cache=bits(c.k_cache), v_cache=bits(c.v_cache),
            block_tables=c.block_tables.numpy(), seq_lens=c.seq_lens.numpy(), cum_seq_lens_q=c.cum_seq_lens_q.numpy(),
            out=bits(out),
        )
        print("wrote", name, tuple(out.shape))


def rope_cases():
    # (name, dtype, shape, x strides or None, algorithm 0 GPT-J / 1 GPT-NeoX, table_len, 2-D position ids)
    # shapes and strides after the reference's own cases (test/infiniop/rope.py:27-38)
    yield "rope_fp16_neox_3d", torch.float16, (10, 32, 64), None, 1, 64, False
    yield "rope_bf16_gptj_3d", torch.bfloat16, (11, 33, 128), None, 0, 48, False
    yield "rope_fp16_gptj_strided", torch.float16, (3, 32, 128), (8000, 200, 1), 0, 32, False
    yield "rope_bf16_neox_4d", torch.bfloat16, (8, 10, 32, 64), None, 1, 40, True
    yield "rope_bf16_neox_4d_permuted", torch.bfloat16, (8, 20, 4, 64), (20 * 4 * 64 * 2, 64, 20 * 64 * 2, 1), 1, 40, False
    yield "rope_f32_neox_3d", torch.float32, (7, 5, 32), None, 1, 16, False
    yield "rope_f32_gptj_3d", torch.float32, (4, 1, 32), (64, 64, 1), 0, 16, False


def strided(shape, strides, dtype, g):
    if strides is None:
        return torch.randn(shape, generator=g).to(dtype)
    extent = 1 + sum((n - 1) * s for n, s in zip(shape, strides))
    return torch.randn(extent, generator=g).to(dtype).as_strided(shape, strides)


def make_rope(ref_rope):
    class _Algo:  # the checker compares against the module's own enum members
        pass

    for idx, (name, dtype, shape, strides, algo, table_len, pos_2d) in enumerate(rope_cases()):
        g = torch.Generator()
        g.manual_seed(300 + idx)
        x = strided(shape, strides, dtype, g)
        seqlen, dhead = shape[-3], shape[-1]
        pos_shape = (shape[0], seqlen) if pos_2d else (seqlen,)
        pos = torch.randint(0, table_len, pos_shape, generator=g, dtype=torch.int64)
        # tables as the reference test builds them (theta 1e5 there; values are rounded to the tensor type)
        freqs = 1.0 / (1e5 ** (torch.arange(0, dhead, 2)[: dhead // 2].float() / dhead))
        angles = torch.outer(torch.arange(table_len).float(), freqs)
        sin_table, cos_table = torch.sin(angles).to(dtype), torch.cos(angles).to(dtype)
        ans = torch.zeros(shape, dtype=dtype)
        # rows of the tables per token, shaped to broadcast over heads as the reference test passes them
        sin_rows, cos_rows = sin_table[pos], cos_table[pos]
        algo_member = ref_rope.Algorithm.GPT_J if algo == 0 else ref_rope.Algorithm.GPT_NEOX
        if x.ndim == 3:
            ref_rope.rotary_embedding(ans, x, sin_rows, cos_rows, 0, algo_member)
        else:
            for b in range(shape[0]):
                rows = (sin_rows[b], cos_rows[b]) if pos_2d else (sin_rows, cos_rows)
                ref_rope.rotary_embedding(ans[b], x[b], rows[0], rows[1], 0, algo_member)
        np.savez_compressed(
            HERE / f"{name}.npz",
            dtype=np.int64(DTYPE_CODE[dtype]), algo=np.int64(algo),
            x=bits(x.contiguous()), x_strides=np.array(strides if strides is not None else [], dtype=np.int64),
            pos_ids=pos.numpy(), sin_table=bits(sin_table), cos_table=bits(cos_table), y=bits(ans),
        )
        print("wrote", name, shape)


def kv_caching_cases():
    # (name, dtype, cache shape, cache strides or None, seq_len): shapes and strides of the reference's own cases
    # (test/infiniop/kv_caching.py:48-56)
    yield "kvc_bf16_8x8x64x32", torch.bfloat16, (8, 8, 64, 32), None, 5
    yield "kvc_fp16_strided_1x32x8x64", torch.float16, (1, 32, 8, 64), (32768, 1024, 64, 1), 3
    yield "kvc_f32_strided_4x8x32x16", torch.float32, (4, 8, 32, 16), (65536, 8192, 256, 16), 7
    yield "kvc_fp16_1x1x8x1", torch.float16, (1, 1, 8, 1), None, 2


def make_kv_caching(ref_kvc):
    for idx, (name, dtype, shape, strides, seq_len) in enumerate(kv_caching_cases()):
        g = torch.Generator()
        g.manual_seed(400 + idx)
        k_cache, v_cache = strided(shape, strides, dtype, g), strided(shape, strides, dtype, g)
        new_shape = (shape[0], shape[1], seq_len, shape[3])
        k, v = torch.randn(new_shape, generator=g).to(dtype), torch.randn(new_shape, generator=g).to(dtype)
        past = torch.randint(0, shape[2] - seq_len + 1, (shape[0],), generator=g, dtype=torch.int64)
        before_k, before_v = bits(k_cache.contiguous()), bits(v_cache.contiguous())
        k_after, v_after = ref_kvc.torch_kv_caching(k_cache, v_cache, k, v, past)
        np.savez_compressed(
            HERE / f"{name}.npz",
            dtype=np.int64(DTYPE_CODE[dtype]), cache_strides=np.array(strides if strides is not None else [], dtype=np.int64),
            k_cache=before_k, v_cache=before_v, k=bits(k), v=bits(v), past_kv_lengths=past.numpy(),
            k_cache_after=bits(k_after.contiguous()), v_cache_after=bits(v_after.contiguous()),
        )
        print("wrote", name, shape)


def layer_cases():
    # (name, case, algorithm): a whole decode layer = the reference's four checkers in the order its callers
    # issue the operators: rotary embedding of q and of the new K row, cache scatter, attention
    yield "layer_bf16_gqa4_hd128_neox", workloads.build_case(
        "x", dtype=torch.bfloat16, seq_lens=[100, 17, 1, 60, 33], num_heads=16, num_kv_heads=4, head_size=128,
        block_size=16, seed=501), 1
    yield "layer_fp16_gqa2_hd64_gptj", workloads.build_case(
        "x", dtype=torch.float16, seq_lens=[64, 5, 100], num_heads=4, num_kv_heads=2, head_size=64,
        block_size=16, seed=502), 0


def make_layers(ref_attn, ref_cache, ref_rope):
    for name, c, algo in layer_cases():
        pos = (c.seq_lens - 1).clamp(min=0)
        table_len = int(pos.max()) + 1
        freqs = 1.0 / (1e4 ** (torch.arange(0, c.head_size, 2).float() / c.head_size))
        angles = torch.outer(torch.arange(table_len).float(), freqs)
        sin_table, cos_table = torch.sin(angles).to(c.dtype), torch.cos(angles).to(c.dtype)
        member = ref_rope.Algorithm.GPT_J if algo == 0 else ref_rope.Algorithm.GPT_NEOX
        q_rot, k_rot = torch.zeros_like(c.q), torch.zeros_like(c.new_k)
        ref_rope.rotary_embedding(q_rot, c.q, sin_table[pos], cos_table[pos], 0, member)
        ref_rope.rotary_embedding(k_rot, c.new_k, sin_table[pos], cos_table[pos], 0, member)
        k_after, v_after = ref_cache.ref_paged_caching(c.k_cache.clone(), c.v_cache.clone(), k_rot, c.new_v, c.slot_mapping)
        out = ref_attn.ref_single_query_cached_kv_attention(q_rot, k_after, v_after, c.block_tables, c.seq_lens, c.scale, None)
        np.savez_compressed(
            HERE / f"{name}.npz",
            dtype=np.int64(DTYPE_CODE[c.dtype]), algo=np.int64(algo), scale=np.float32(c.scale),
            q=bits(c.q), k_cache=bits(c.k_cache), v_cache=bits(c.v_cache), new_k=bits(c.new_k), new_v=bits(c.new_v),
            slot_mapping=c.slot_mapping.numpy(), block_tables=c.block_tables.numpy(), seq_lens=c.seq_lens.numpy(),
            pos_ids=pos.numpy(), sin_table=bits(sin_table), cos_table=bits(cos_table),
            q_rot=bits(q_rot), k_cache_after=bits(k_after), v_cache_after=bits(v_after), out=bits(out),
        )
        print("wrote", name, tuple(out.shape))


def main():
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    only = [a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--only=")]
    ref_arg = args[0] if args else os.getenv("INFINICORE_REFERENCE")
    if not ref_arg:
        raise SystemExit("usage: make_golden.py <reference checkout> [--only=...]  (or set INFINICORE_REFERENCE)")
    ref_root = Path(ref_arg)
    ref_attn, ref_cache, ref_prefill, ref_rope, ref_kvc = load_reference(ref_root)
    torch.set_num_threads(4)
    if not only or "attention" in only:
        make_attention(ref_attn)
    if not only or "caching" in only:
        make_caching(ref_cache)
    if not only or "prefill" in only:
        make_prefill(ref_prefill)
    if not only or "rope" in only:
        make_rope(ref_rope)
    if not only or "kv_caching" in only:
        make_kv_caching(ref_kvc)
    if not only or "layer" in only:
        make_layers(ref_attn, ref_cache, ref_rope)


if __name__ == "__main__":
    main()
