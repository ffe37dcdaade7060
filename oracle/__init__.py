"""TEST INFRASTRUCTURE - CPU oracle for the paged decode path.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this package.
It wraps oracle/paged_oracle.c (a restatement of the reference's torch checkers, see the
header of that file) and oracle/rope_oracle.c (the reference's CPU rotary embedding) for numpy
arrays holding raw 16-bit patterns.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_double, c_float, c_int, c_int64, c_ssize_t, c_uint16, c_void_p

import numpy as np

from .build import build as _build

F16, F32, F64, BF16 = 12, 13, 14, 19

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(_build()))
        _lib.oracle_paged_attention.restype = c_int
        _lib.oracle_paged_attention.argtypes = [
            c_int, c_int, c_void_p,
            c_void_p, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t,
            c_void_p,
            c_void_p,
            c_float,
            c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
        ]
        _lib.oracle_paged_attention_prefill.restype = c_int
        _lib.oracle_paged_attention_prefill.argtypes = [
            c_int, c_int, c_void_p,
            c_void_p, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t,
            c_void_p, c_void_p,
            c_void_p,
            c_float,
            c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
        ]
        _lib.oracle_paged_caching.restype = c_int
        _lib.oracle_paged_caching.argtypes = [
            c_int64,
            c_void_p, c_ssize_t, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t, c_ssize_t,
            c_void_p,
            c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
        ]
        _lib.oracle_float_to_f16.restype = c_uint16
        _lib.oracle_float_to_f16.argtypes = [c_float]
        _lib.oracle_float_to_bf16.restype = c_uint16
        _lib.oracle_float_to_bf16.argtypes = [c_float]
        _lib.oracle_f16_to_float.restype = c_float
        _lib.oracle_f16_to_float.argtypes = [c_uint16]
        _lib.oracle_bf16_to_float.restype = c_float
        _lib.oracle_bf16_to_float.argtypes = [c_uint16]
        _lib.oracle_num_threads.restype = c_int
        _lib.oracle_set_num_threads.restype = c_int
        _lib.oracle_set_num_threads.argtypes = [c_int]
        _lib.oracle_rope.restype = c_int
        _lib.oracle_rope.argtypes = [
            c_int, c_int,
            c_void_p, c_ssize_t, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t, c_ssize_t, c_ssize_t,
            c_void_p, c_ssize_t,
            c_void_p, c_void_p,
            c_int64, c_int64, c_int64, c_int64, c_int64,
        ]
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Lets the oracle's OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS a
    launcher exported (torch.distributed.run sets it to 1 for its workers).  Returns the thread count."""
    import os

    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    return int(lib().oracle_set_num_threads(cores))


def _elem_strides(a: np.ndarray):
    assert all(s % a.itemsize == 0 for s in a.strides)
    return [s // a.itemsize for s in a.strides]


def paged_attention(q, k_cache, v_cache, block_tables, seq_lens, scale, dtype, alibi_slopes=None,
                    mode="exact", out=None) -> np.ndarray:
    """q/k_cache/v_cache: uint16 arrays of raw F16/BF16 bits (any strides, last dim dense).
    Returns float64 [num_seqs, num_heads, value_size]; rows of empty sequences keep the
    values of `out` (NaN when `out` is not given)."""
    assert q.dtype == np.uint16 and k_cache.dtype == np.uint16 and v_cache.dtype == np.uint16
    num_seqs, num_heads, head_size = q.shape
    num_blocks, num_kv_heads, block_size, _ = k_cache.shape
    value_size = v_cache.shape[3]
    bt = np.ascontiguousarray(block_tables, dtype=np.int64)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int64)
    if out is None:
        out = np.full((num_seqs, num_heads, value_size), np.nan, dtype=np.float64)
    assert out.dtype == np.float64 and out.flags.c_contiguous
    qs, ks, vs = _elem_strides(q), _elem_strides(k_cache), _elem_strides(v_cache)
    assert qs[2] == 1 and ks[3] == 1 and vs[3] == 1
    al = None
    if alibi_slopes is not None:
        al = np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    rc = lib().oracle_paged_attention(
        0 if mode == "exact" else 1, int(dtype), out.ctypes.data,
        q.ctypes.data, qs[0], qs[1],
        k_cache.ctypes.data, ks[0], ks[1], ks[2],
        v_cache.ctypes.data, vs[0], vs[1], vs[2],
        bt.ctypes.data, bt.shape[1] if bt.ndim == 2 else 0,
        sl.ctypes.data,
        al.ctypes.data if al is not None else None,
        float(scale),
        num_seqs, num_heads, num_kv_heads, head_size, value_size, block_size, num_blocks, bt.shape[1],
    )
    if rc != 0:
        raise ValueError(f"oracle_paged_attention rejected its input (code {rc})")
    return out


def paged_attention_prefill(q, k_cache, v_cache, block_tables, seq_lens, cum_seq_lens_q, scale, dtype,
                            alibi_slopes=None, mode="exact", out=None) -> np.ndarray:
    """q: uint16 [total_q, num_heads, head_size] packed over sequences.  Returns float64
    [total_q, num_heads, value_size]; rows outside every chunk keep `out` (NaN when not given)."""
    assert q.dtype == np.uint16 and k_cache.dtype == np.uint16 and v_cache.dtype == np.uint16
    total_q, num_heads, head_size = q.shape
    num_blocks, num_kv_heads, block_size, _ = k_cache.shape
    value_size = v_cache.shape[3]
    bt = np.ascontiguousarray(block_tables, dtype=np.int64)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int64)
    cq = np.ascontiguousarray(cum_seq_lens_q, dtype=np.int64)
    assert cq.shape[0] == sl.shape[0] + 1
    if out is None:
        out = np.full((total_q, num_heads, value_size), np.nan, dtype=np.float64)
    assert out.dtype == np.float64 and out.flags.c_contiguous
    qs, ks, vs = _elem_strides(q), _elem_strides(k_cache), _elem_strides(v_cache)
    assert qs[2] == 1 and ks[3] == 1 and vs[3] == 1
    al = None
    if alibi_slopes is not None:
        al = np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    rc = lib().oracle_paged_attention_prefill(
        0 if mode == "exact" else 1, int(dtype), out.ctypes.data,
        q.ctypes.data, qs[0], qs[1],
        k_cache.ctypes.data, ks[0], ks[1], ks[2],
        v_cache.ctypes.data, vs[0], vs[1], vs[2],
        bt.ctypes.data, bt.shape[1],
        sl.ctypes.data, cq.ctypes.data,
        al.ctypes.data if al is not None else None,
        float(scale),
        sl.shape[0], num_heads, num_kv_heads, head_size, value_size, block_size, num_blocks, bt.shape[1],
    )
    if rc != 0:
        raise ValueError(f"oracle_paged_attention_prefill rejected its input (code {rc})")
    return out


def paged_caching(k_cache, v_cache, k, v, slot_mapping) -> None:
    """In-place, byte-exact scatter of k/v rows into the pools (arrays of any 2- or 4-byte dtype)."""
    es = k_cache.itemsize
    assert v_cache.itemsize == es and k.itemsize == es and v.itemsize == es
    num_blocks, num_kv_heads, block_size, head_size = k_cache.shape[:4]
    v_head_size = v_cache.shape[3]
    sm = np.ascontiguousarray(slot_mapping, dtype=np.int64)
    kcs, vcs, ks, vs = (_elem_strides(a) for a in (k_cache, v_cache, k, v))
    assert kcs[3] == 1 and vcs[3] == 1 and ks[2] == 1 and vs[2] == 1
    rc = lib().oracle_paged_caching(
        es,
        k_cache.ctypes.data, kcs[0], kcs[1], kcs[2],
        v_cache.ctypes.data, vcs[0], vcs[1], vcs[2],
        k.ctypes.data, ks[0], ks[1],
        v.ctypes.data, vs[0], vs[1],
        sm.ctypes.data,
        sm.shape[0], num_kv_heads, head_size, v_head_size, block_size, num_blocks,
    )
    if rc != 0:
        raise ValueError(f"oracle_paged_caching rejected its input (code {rc})")


def rope(x, pos_ids, sin_table, cos_table, dtype, gpt_j, out=None) -> np.ndarray:
    """x: [seqlen, nhead, dhead] or [batch, seqlen, nhead, dhead]; uint16 bit patterns for F16 / BF16,
    float32 / float64 otherwise (any strides, last dim dense).  pos_ids: [seqlen] or [batch, seqlen].
    Tables: [table_len, dhead / 2] in the same representation.  Returns `out` (a new dense array when
    not given; `out` may be `x` itself)."""
    want = {F16: np.uint16, BF16: np.uint16, F32: np.float32, F64: np.float64}[int(dtype)]
    assert x.dtype == want and sin_table.dtype == want and cos_table.dtype == want
    sin_table = np.ascontiguousarray(sin_table)
    cos_table = np.ascontiguousarray(cos_table)
    if out is None:
        out = np.empty(x.shape, dtype=want)
    assert out.shape == x.shape and out.dtype == want
    x4 = x if x.ndim == 4 else x[None]
    y4 = out if out.ndim == 4 else out[None]
    batch, seqlen, nhead, dhead = x4.shape
    table_len, table_dim = sin_table.shape
    assert dhead == 2 * table_dim and cos_table.shape == sin_table.shape
    pos = np.ascontiguousarray(pos_ids, dtype=np.int64)
    assert pos.shape in ((seqlen,), (batch, seqlen))
    xs, ys = _elem_strides(x4), _elem_strides(y4)
    assert xs[3] == 1 and ys[3] == 1
    rc = lib().oracle_rope(
        int(dtype), 1 if gpt_j else 0,
        y4.ctypes.data, ys[0], ys[1], ys[2],
        x4.ctypes.data, xs[0], xs[1], xs[2],
        pos.ctypes.data, seqlen if pos.ndim == 2 else 0,
        sin_table.ctypes.data, cos_table.ctypes.data,
        batch, seqlen, nhead, table_dim, table_len,
    )
    if rc != 0:
        raise ValueError(f"oracle_rope rejected its input (code {rc})")
    return out


def kv_caching(k_cache, v_cache, k, v, past_kv_lengths) -> None:
    """In-place restatement of the reference checker torch_kv_caching (test/infiniop/kv_caching.py:25-41) and of
    its kernel's indexing (src/infiniop/ops/kv_caching/cuda/kernel.cuh:32-60) for numpy arrays of any dtype and
    strides: cache[b, h, past[b] + s, :] = new[b, h, s, :].  Rows whose destination lies outside the cache are
    skipped (the checker's slice assignment would raise, the reference kernel writes out of bounds)."""
    batch, heads, max_len, _ = k_cache.shape
    seq_len = k.shape[2]
    past = np.asarray(past_kv_lengths).astype(np.int64)
    for b in range(batch):
        for s in range(seq_len):
            dst = int(past[b]) + s
            if 0 <= dst < max_len:
                k_cache[b, :, dst, :] = k[b, :, s, :]
                v_cache[b, :, dst, :] = v[b, :, s, :]
