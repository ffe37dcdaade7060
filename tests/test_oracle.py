"""CPU tests that pin the oracle (oracle/paged_oracle.c) to the reference.

The golden files hold outputs of the reference's own torch checkers
(ref_single_query_cached_kv_attention, ref_paged_caching) on seeded inputs - see
tests/golden/make_golden.py.  The oracle's "reference" mode reproduces those roundings and must
agree to within a couple of output ulps (summation order is the only freedom); its "exact" mode
must agree within the path's parity tolerance.
"""
import numpy as np
import pytest

import oracle
from helpers import ATTN_TOL, BF16, F16, bits_to_float, golden_names, load_golden


def _ulp(dtype_code, x):
    mant = 10 if dtype_code == F16 else 7
    return np.maximum(np.abs(x), 2.0 ** -14) * 2.0 ** -mant


@pytest.mark.parametrize("name", golden_names("attn_"))
def test_attention_reference_mode_matches_reference_output(name):
    g = load_golden(name)
    dt = int(g["dtype"])
    alibi = g["alibi"] if g["alibi"].size else None
    got = oracle.paged_attention(g["q"], g["k_cache"], g["v_cache"], g["block_tables"], g["seq_lens"],
                                 float(g["scale"]), dt, alibi, mode="reference")
    want = bits_to_float(g["out"], dt)
    # Same roundings, different summation order: a rounded score or probability can flip by one ulp of the
    # tensor type.  For an output element of ordinary size that is a few of ITS ulps (first term); an
    # element that is a near-cancellation of large terms moves by a flip's share of those terms instead,
    # which is measured against the largest output, not against the element (second term).  Observed on
    # the committed vectors: 99.87 % of all elements within one ulp, the worst 4.9 of its own ulps and
    # 2.7e-4 of the largest output; four of the eight vectors match bit for bit.
    err = np.abs(got - want)
    assert np.all(err <= 4 * _ulp(dt, want) + 5e-4 * np.abs(want).max()), f"max err {err.max():.3e}"
    assert np.mean(err <= _ulp(dt, want)) > 0.998


@pytest.mark.parametrize("name", golden_names("attn_"))
def test_attention_exact_mode_within_path_tolerance(name):
    g = load_golden(name)
    dt = int(g["dtype"])
    alibi = g["alibi"] if g["alibi"].size else None
    got = oracle.paged_attention(g["q"], g["k_cache"], g["v_cache"], g["block_tables"], g["seq_lens"],
                                 float(g["scale"]), dt, alibi, mode="exact")
    want = bits_to_float(g["out"], dt)
    atol, rtol = ATTN_TOL[dt]
    assert np.all(np.abs(got - want) <= atol + rtol * np.abs(want))


@pytest.mark.parametrize("name", golden_names("cache_"))
def test_caching_bit_exact_against_reference_output(name):
    g = load_golden(name)
    k_cache, v_cache = g["k_cache"].copy(), g["v_cache"].copy()
    if int(g["permuted"]):
        # stored physically as [blocks, slots, heads, dim]; the operator sees [blocks, heads, slots, dim]
        oracle.paged_caching(k_cache.transpose(0, 2, 1, 3), v_cache.transpose(0, 2, 1, 3), g["k"], g["v"], g["slot_mapping"])
    else:
        oracle.paged_caching(k_cache, v_cache, g["k"], g["v"], g["slot_mapping"])
    assert np.array_equal(k_cache, g["k_cache_after"])
    assert np.array_equal(v_cache, g["v_cache_after"])


def test_caching_skips_negative_slots_and_rejects_out_of_pool():
    rng = np.random.default_rng(0)
    k_cache = rng.integers(0, 65536, (4, 2, 16, 64), dtype=np.uint16)
    v_cache = rng.integers(0, 65536, (4, 2, 16, 64), dtype=np.uint16)
    k = rng.integers(0, 65536, (3, 2, 64), dtype=np.uint16)
    v = rng.integers(0, 65536, (3, 2, 64), dtype=np.uint16)
    before = k_cache.copy()
    oracle.paged_caching(k_cache, v_cache, k, v, np.array([5, -1, 40]))
    assert np.array_equal(k_cache[0, :, 5], k[0]) and np.array_equal(k_cache[2, :, 8], k[2])
    mask = np.ones_like(before, dtype=bool)
    mask[0, :, 5] = False
    mask[2, :, 8] = False
    assert np.array_equal(k_cache[mask], before[mask])
    with pytest.raises(ValueError):
        oracle.paged_caching(k_cache, v_cache, k, v, np.array([5, 6, 64]))


def test_attention_leaves_empty_sequences_untouched():
    g = load_golden("attn_bf16_gqa4_hd128")
    lens = g["seq_lens"].copy()
    lens[1] = 0
    out = np.full((4, 8, 128), 7.0)
    oracle.paged_attention(g["q"], g["k_cache"], g["v_cache"], g["block_tables"], lens, float(g["scale"]), BF16, out=out)
    assert np.all(out[1] == 7.0) and not np.any(out[0] == 7.0)


def test_codecs_round_trip_every_finite_pattern():
    lib = oracle.lib()
    for h in list(range(0, 0x7c00, 7)) + [0x7bff, 0x0001, 0x03ff, 0x0400, 0x8001, 0xfbff]:
        assert lib.oracle_float_to_f16(lib.oracle_f16_to_float(h)) == h
    for h in list(range(0, 0x7f80, 13)) + [0x7f7f, 0x0001, 0x8001]:
        assert lib.oracle_float_to_bf16(lib.oracle_bf16_to_float(h)) == h
    # ties go to even
    assert lib.oracle_float_to_f16(1.0 + 2.0 ** -11) == 0x3c00
    assert lib.oracle_float_to_f16(1.0 + 3 * 2.0 ** -11) == 0x3c02
    assert lib.oracle_float_to_bf16(1.0 + 2.0 ** -8) == 0x3f80
    assert lib.oracle_float_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3f82


# ---- prefill ------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", golden_names("prefill_"))
def test_prefill_reference_mode_matches_reference_output(name):
    g = load_golden(name)
    dt = int(g["dtype"])
    got = oracle.paged_attention_prefill(g["q"], g["k_cache"], g["v_cache"], g["block_tables"], g["seq_lens"],
                                         g["cum_seq_lens_q"], float(g["scale"]), dt, mode="reference")
    want = bits_to_float(g["out"], dt)
    err = np.abs(got - want)
    assert np.all(err <= 4 * _ulp(dt, want) + 1e-3 * np.abs(want).max()), f"max err {err.max():.3e}"
    assert np.mean(err <= _ulp(dt, want)) > 0.9


@pytest.mark.parametrize("name", golden_names("prefill_"))
def test_prefill_exact_mode_within_path_tolerance(name):
    g = load_golden(name)
    dt = int(g["dtype"])
    got = oracle.paged_attention_prefill(g["q"], g["k_cache"], g["v_cache"], g["block_tables"], g["seq_lens"],
                                         g["cum_seq_lens_q"], float(g["scale"]), dt, mode="exact")
    want = bits_to_float(g["out"], dt)
    atol, rtol = ATTN_TOL[dt]
    assert np.all(np.abs(got - want) <= atol + rtol * np.abs(want))


def test_prefill_row_equals_decode_with_the_causal_length():
    """A new token is a decode query against the first cached + t + 1 tokens: the two oracles agree bit for bit."""
    g = load_golden("prefill_bf16_mha_hd128")
    dt = int(g["dtype"])
    full = oracle.paged_attention_prefill(g["q"], g["k_cache"], g["v_cache"], g["block_tables"], g["seq_lens"],
                                          g["cum_seq_lens_q"], float(g["scale"]), dt)
    cum, lens = g["cum_seq_lens_q"], g["seq_lens"]
    for s in range(len(lens)):
        n = cum[s + 1] - cum[s]
        for t in (0, n // 2, n - 1):
            row = cum[s] + t
            dec = oracle.paged_attention(g["q"][row:row + 1], g["k_cache"], g["v_cache"], g["block_tables"][s:s + 1],
                                         np.array([lens[s] - n + t + 1]), float(g["scale"]), dt)
            assert np.array_equal(dec[0], full[row])


# ---- rotary embedding -----------------------------------------------------------------------------------


def _rope_inputs(g):
    x = g["x"]
    if g["x_strides"].size:  # rebuild the strided layout the fixture was generated with
        strides = [int(s) for s in g["x_strides"]]
        extent = 1 + sum((n - 1) * s for n, s in zip(x.shape, strides))
        base = np.zeros(extent, dtype=x.dtype)
        view = np.lib.stride_tricks.as_strided(base, x.shape, [s * x.itemsize for s in strides])
        view[...] = x
        x = view
    return x


@pytest.mark.parametrize("name", golden_names("rope_"))
def test_rope_bit_exact_against_reference_checker(name):
    g = load_golden(name)
    x = _rope_inputs(g)
    got = oracle.rope(x, g["pos_ids"], g["sin_table"], g["cos_table"], int(g["dtype"]), int(g["algo"]) == 0)
    assert np.array_equal(got, g["y"])
    # in place, as half of the reference's test cases run it
    oracle.rope(x, g["pos_ids"], g["sin_table"], g["cos_table"], int(g["dtype"]), int(g["algo"]) == 0, out=x)
    assert np.array_equal(np.ascontiguousarray(x), g["y"])


def test_rope_is_a_rotation_and_positions_outside_the_tables_copy():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((6, 3, 32))
    ang = rng.uniform(0, 6.28, (10, 16))
    pos = np.array([0, 9, 3, -1, 10, 5])
    for gpt_j in (True, False):
        y = oracle.rope(x, pos, np.sin(ang), np.cos(ang), oracle.F64, gpt_j)
        assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1), rtol=1e-12)      # pairs keep their norm
        assert np.array_equal(y[3], x[3]) and np.array_equal(y[4], x[4])        # -1 and 10 are outside a table of 10 rows
        back = oracle.rope(y, pos, -np.sin(ang), np.cos(ang), oracle.F64, gpt_j)  # the inverse rotation
        assert np.allclose(back, x, atol=1e-12)


# ---- contiguous KV cache append -------------------------------------------------------------------------


def _strided_np(dense, strides):
    if not len(strides):
        return dense.copy()
    strides = [int(s) for s in strides]
    extent = 1 + sum((n - 1) * s for n, s in zip(dense.shape, strides))
    base = np.zeros(extent, dtype=dense.dtype)
    view = np.lib.stride_tricks.as_strided(base, dense.shape, [s * dense.itemsize for s in strides])
    view[...] = dense
    return view


@pytest.mark.parametrize("name", golden_names("kvc_"))
def test_kv_caching_bit_exact_against_reference_checker(name):
    g = load_golden(name)
    kc, vc = _strided_np(g["k_cache"], g["cache_strides"]), _strided_np(g["v_cache"], g["cache_strides"])
    oracle.kv_caching(kc, vc, g["k"], g["v"], g["past_kv_lengths"])
    assert np.array_equal(np.ascontiguousarray(kc), g["k_cache_after"])
    assert np.array_equal(np.ascontiguousarray(vc), g["v_cache_after"])


def test_kv_caching_skips_rows_outside_the_cache():
    kc, vc = np.zeros((2, 1, 4, 2), np.float32), np.zeros((2, 1, 4, 2), np.float32)
    k = np.arange(12, dtype=np.float32).reshape(2, 1, 3, 2) + 1
    oracle.kv_caching(kc, vc, k, -k, np.array([2, -1]))
    assert np.array_equal(kc[0, 0], [[0, 0], [0, 0], [1, 2], [3, 4]])          # third row would land at 4: skipped
    assert np.array_equal(kc[1, 0], [[9, 10], [11, 12], [0, 0], [0, 0]])       # first row would land at -1: skipped
    assert np.array_equal(vc, -kc)


# ---- a whole decode layer: rotary embedding of q and the new K row, scatter, attention --------------------


@pytest.mark.parametrize("name", golden_names("layer_"))
def test_decode_layer_composition_matches_the_reference_checkers(name):
    """The four oracle functions chained as a decode layer chains the operators, against the same chain of the
    reference's own checkers: rotated rows and caches bit for bit, attention as in the attention tests."""
    g = load_golden(name)
    dt, gpt_j = int(g["dtype"]), int(g["algo"]) == 0
    q_rot = oracle.rope(g["q"], g["pos_ids"], g["sin_table"], g["cos_table"], dt, gpt_j)
    k_rot = oracle.rope(g["new_k"], g["pos_ids"], g["sin_table"], g["cos_table"], dt, gpt_j)
    assert np.array_equal(q_rot, g["q_rot"])
    kc, vc = g["k_cache"].copy(), g["v_cache"].copy()
    oracle.paged_caching(kc, vc, k_rot, g["new_v"], g["slot_mapping"])
    assert np.array_equal(kc, g["k_cache_after"]) and np.array_equal(vc, g["v_cache_after"])
    got = oracle.paged_attention(q_rot, kc, vc, g["block_tables"], g["seq_lens"], float(g["scale"]), dt, None, mode="reference")
    want = bits_to_float(g["out"], dt)
    err = np.abs(got - want)
    assert np.all(err <= 4 * _ulp(dt, want) + 1e-3 * np.abs(want).max()), f"max err {err.max():.3e}"
