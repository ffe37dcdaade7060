"""User-facing operators on torch CUDA tensors, routed through the C ABI.

Same names, argument order and meaning as the reference's Python operators
(python/infinicore/ops/paged_attention.py:5-41, python/infinicore/ops/paged_caching.py:5-22);
descriptor reuse follows the reference's per-thread, per-device LRU keyed on tensor metadata
(src/infinicore/ops/infiniop_impl.hpp:8-78, capacity 100).  torch supplies device memory and the
current stream; every byte of compute happens inside libinfiniop.
"""
from __future__ import annotations

import ctypes
import threading
from collections import OrderedDict

import torch

from .libinfiniop import (
    LIBINFINIOP, InfiniDeviceEnum, InfiniDtype, TestTensor, check_error, create_handle,
    infiniopOperatorDescriptor_t, to_infini_dtype,
)

_CACHE_CAPACITY = 100
_tls = threading.local()


def _state(device_index: int):
    per_dev = getattr(_tls, "per_dev", None)
    if per_dev is None:
        per_dev = _tls.per_dev = {}
    st = per_dev.get(device_index)
    if st is None:
        check_error(LIBINFINIOP.infinirtSetDevice(InfiniDeviceEnum.NVIDIA, device_index))
        st = per_dev[device_index] = {"handle": create_handle(), "cache": OrderedDict(), "workspace": {}}
    else:
        # infinirt's current device is per host thread; keep it in step with the tensors' device
        check_error(LIBINFINIOP.infinirtSetDevice(InfiniDeviceEnum.NVIDIA, device_index))
    return st


WAIT_EXPIRED, BLOCK_OUT_OF_RANGE, SLOT_OUT_OF_RANGE = 1, 2, 4


def kernel_status(device=None, stream=None) -> int:
    """Waits for `stream` (default: torch's current stream on `device`) and returns the device's word of
    kernel status flags, clearing it: 0 when every kernel of this library did all of its work, else a
    combination of WAIT_EXPIRED (a worker gave up waiting for one of its own copies: output rows are
    missing), BLOCK_OUT_OF_RANGE and SLOT_OUT_OF_RANGE (index checking, switched on with
    INFINIOP_PAGED_CHECK_INDICES=1 when a descriptor is created, met an index outside the pool).
    No counterpart in the reference, whose kernels report nothing."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    st = _state(dev)
    sptr = torch.cuda.current_stream(dev).cuda_stream if stream is None else int(stream)
    flags = ctypes.c_uint32(0)
    check_error(LIBINFINIOP.infiniopGetKernelStatus(st["handle"], ctypes.c_void_p(sptr), ctypes.byref(flags)))
    return int(flags.value)


def _meta(t, index_dtype=None):
    if t is None:
        return None
    return (index_dtype or str(t.dtype), tuple(t.shape), tuple(t.stride()))


def _desc(t: torch.Tensor, dt=None):
    return TestTensor.from_torch(t, dt if dt is not None else to_infini_dtype(t.dtype), InfiniDeviceEnum.NVIDIA)


def _require_cuda(*tensors):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("infinicore_b200 operators run on CUDA tensors only; there is no CPU fallback")
        dev = t.device.index if dev is None else dev
        if t.device.index != dev:
            raise RuntimeError("all tensors of one call must live on the same GPU")
    return dev


def _lookup(st, key, make):
    cache = st["cache"]
    entry = cache.get(key)
    if entry is None:
        entry = make()
        cache[key] = entry
        if len(cache) > _CACHE_CAPACITY:
            _, old = cache.popitem(last=False)
            old["destroy"](old["desc"])
    else:
        cache.move_to_end(key)
    return entry


def _workspace(st, nbytes: int, device_index: int):
    """One grow-only scratch buffer per (thread, device, stream)."""
    if nbytes == 0:
        return None
    stream = torch.cuda.current_stream(device_index).cuda_stream
    buf = st["workspace"].get(stream)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{device_index}")
        st["workspace"][stream] = buf
    return buf


def paged_attention(q, k_cache, v_cache, block_tables, cache_lens, alibi_slopes=None, scale: float = 1.0, *, out=None):
    """Decode attention of one query token per sequence over a paged KV cache.

    q [num_seqs, num_heads, head_size]; k_cache/v_cache [num_blocks, num_kv_heads, block_size,
    head_size]; block_tables [num_seqs, max_blocks] and cache_lens [num_seqs] int64 or int32.
    Returns `out` (allocated when not given).  `out` may also be a PINNED HOST tensor: page-locked memory is
    mapped into the device's address space, so the kernels store the output rows over PCIe themselves and no
    device-to-host copy is needed afterwards (valid once the stream has been synchronised)."""
    host_out = out is not None and not out.is_cuda and out.is_pinned()
    dev = _require_cuda(q, k_cache, v_cache, block_tables, cache_lens, alibi_slopes, None if host_out else out)
    if out is None:
        out = torch.empty((*q.shape[:-1], v_cache.shape[3]), dtype=q.dtype, device=q.device)
    st = _state(dev)
    key = ("paged_attention", _meta(out), _meta(q), _meta(k_cache), _meta(v_cache), _meta(block_tables),
           _meta(cache_lens), _meta(alibi_slopes), float(scale))

    def make():
        tensors = [_desc(out), _desc(q), _desc(k_cache), _desc(v_cache), _desc(block_tables), _desc(cache_lens)]
        alibi = _desc(alibi_slopes) if alibi_slopes is not None else None
        desc = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedAttentionDescriptor(
            st["handle"], ctypes.byref(desc), *[t.descriptor for t in tensors],
            alibi.descriptor if alibi is not None else None, scale))
        size = ctypes.c_size_t(0)
        check_error(LIBINFINIOP.infiniopGetPagedAttentionWorkspaceSize(desc, ctypes.byref(size)))
        for t in tensors + ([alibi] if alibi is not None else []):
            t.destroy_desc()
        return {"desc": desc, "workspace": size.value, "destroy": LIBINFINIOP.infiniopDestroyPagedAttentionDescriptor}

    entry = _lookup(st, key, make)
    ws = _workspace(st, entry["workspace"], dev)
    with torch.cuda.device(dev):
        check_error(LIBINFINIOP.infiniopPagedAttention(
            entry["desc"], ws.data_ptr() if ws is not None else None, entry["workspace"],
            out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            block_tables.data_ptr(), cache_lens.data_ptr(),
            alibi_slopes.data_ptr() if alibi_slopes is not None else None,
            torch.cuda.current_stream(dev).cuda_stream))
    return out


def paged_attention_multi_out(outs, q, k_cache, v_cache, block_tables, cache_lens, alibi_slopes=None, scale: float = 1.0):
    """paged_attention with every output row stored to several buffers (no reference counterpart).

    `outs[0]` is a tensor [num_seqs, num_heads, head_size] (it may be a strided view, e.g. a head slice
    of a wider tensor); the further entries are tensors of the same shape and strides or raw device
    addresses (ints) of such buffers - for instance the same head slice inside other ranks' outputs in
    symmetric memory.  Returns outs[0]."""
    out = outs[0]
    dev = _require_cuda(q, k_cache, v_cache, block_tables, cache_lens, alibi_slopes, out)
    st = _state(dev)
    key = ("paged_attention", _meta(out), _meta(q), _meta(k_cache), _meta(v_cache), _meta(block_tables),
           _meta(cache_lens), _meta(alibi_slopes), float(scale))

    def make():
        tensors = [_desc(out), _desc(q), _desc(k_cache), _desc(v_cache), _desc(block_tables), _desc(cache_lens)]
        alibi = _desc(alibi_slopes) if alibi_slopes is not None else None
        desc = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedAttentionDescriptor(
            st["handle"], ctypes.byref(desc), *[t.descriptor for t in tensors],
            alibi.descriptor if alibi is not None else None, scale))
        size = ctypes.c_size_t(0)
        check_error(LIBINFINIOP.infiniopGetPagedAttentionWorkspaceSize(desc, ctypes.byref(size)))
        for t in tensors + ([alibi] if alibi is not None else []):
            t.destroy_desc()
        return {"desc": desc, "workspace": size.value, "destroy": LIBINFINIOP.infiniopDestroyPagedAttentionDescriptor}

    entry = _lookup(st, key, make)
    ws = _workspace(st, entry["workspace"], dev)
    ptrs = []
    for o in outs:
        if isinstance(o, torch.Tensor):
            if tuple(o.shape) != tuple(out.shape) or o.stride() != out.stride() or o.dtype != out.dtype:
                raise ValueError("every destination must have the shape, strides and dtype of outs[0]")
            ptrs.append(o.data_ptr())
        else:
            ptrs.append(int(o))
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    with torch.cuda.device(dev):
        check_error(LIBINFINIOP.infiniopPagedAttentionMultiOut(
            entry["desc"], ws.data_ptr() if ws is not None else None, entry["workspace"], arr, len(ptrs),
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(), cache_lens.data_ptr(),
            alibi_slopes.data_ptr() if alibi_slopes is not None else None,
            torch.cuda.current_stream(dev).cuda_stream))
    return out


def paged_attention_prefill(q, k_cache, v_cache, block_tables, history_lens, cu_seqlens_q, alibi_slopes=None,
                            scale: float = 1.0, *, out=None):
    """Causal attention of packed new tokens q [total_q, num_heads, head_size] over each sequence's paged
    KV cache (which already holds the new tokens).  `history_lens` [num_seqs] is the total KV length per
    sequence, `cu_seqlens_q` [num_seqs + 1] the prefix sum of new-token counts; same argument order as
    the reference's python/infinicore/ops/paged_attention_prefill.py:5-46."""
    dev = _require_cuda(q, k_cache, v_cache, block_tables, history_lens, cu_seqlens_q, alibi_slopes, out)
    if out is None:
        out = torch.empty((*q.shape[:-1], v_cache.shape[3]), dtype=q.dtype, device=q.device)
    st = _state(dev)
    key = ("paged_attention_prefill", _meta(out), _meta(q), _meta(k_cache), _meta(v_cache), _meta(block_tables),
           _meta(history_lens), _meta(cu_seqlens_q), _meta(alibi_slopes), float(scale))

    def make():
        tensors = [_desc(out), _desc(q), _desc(k_cache), _desc(v_cache), _desc(block_tables), _desc(history_lens), _desc(cu_seqlens_q)]
        alibi = _desc(alibi_slopes) if alibi_slopes is not None else None
        desc = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedAttentionPrefillDescriptor(
            st["handle"], ctypes.byref(desc), *[t.descriptor for t in tensors],
            alibi.descriptor if alibi is not None else None, scale))
        size = ctypes.c_size_t(0)
        check_error(LIBINFINIOP.infiniopGetPagedAttentionPrefillWorkspaceSize(desc, ctypes.byref(size)))
        for t in tensors + ([alibi] if alibi is not None else []):
            t.destroy_desc()
        return {"desc": desc, "workspace": size.value, "destroy": LIBINFINIOP.infiniopDestroyPagedAttentionPrefillDescriptor}

    entry = _lookup(st, key, make)
    ws = _workspace(st, entry["workspace"], dev)
    with torch.cuda.device(dev):
        check_error(LIBINFINIOP.infiniopPagedAttentionPrefill(
            entry["desc"], ws.data_ptr() if ws is not None else None, entry["workspace"],
            out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
            history_lens.data_ptr(), cu_seqlens_q.data_ptr(),
            alibi_slopes.data_ptr() if alibi_slopes is not None else None,
            torch.cuda.current_stream(dev).cuda_stream))
    return out


class RopeAlgo:
    """Pairing of the rotary embedding (reference python/infinicore/nn/functional/rope.py:5-9)."""

    GPT_J = 0
    GPT_NEOX = 1


def rope(x, pos_ids, sin_table, cos_table, algo: int = RopeAlgo.GPT_NEOX, *, out=None):
    """Rotary position embedding (same signature as the reference's python/infinicore/nn/functional/rope.py:12-45):
    x [seqlen, nhead, dhead] or [batch, seqlen, nhead, dhead], pos_ids [seqlen] or [batch, seqlen] (any integer
    type), tables [table_len, dhead / 2] in x's dtype.  Returns `out` (a new tensor when not given; may be x)."""
    dev = _require_cuda(x, pos_ids, sin_table, cos_table, out)
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    st = _state(dev)
    key = ("rope", _meta(out), _meta(x), _meta(pos_ids), _meta(sin_table), _meta(cos_table), int(algo))

    def make():
        tensors = [_desc(out), _desc(x), _desc(pos_ids), _desc(sin_table), _desc(cos_table)]
        desc = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreateRoPEDescriptor(
            st["handle"], ctypes.byref(desc), *[t.descriptor for t in tensors], int(algo)))
        for t in tensors:
            t.destroy_desc()
        return {"desc": desc, "workspace": 0, "destroy": LIBINFINIOP.infiniopDestroyRoPEDescriptor}

    entry = _lookup(st, key, make)
    with torch.cuda.device(dev):
        check_error(LIBINFINIOP.infiniopRoPE(
            entry["desc"], None, 0, out.data_ptr(), x.data_ptr(), pos_ids.data_ptr(), sin_table.data_ptr(),
            cos_table.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
    return out


def paged_decode_step(q, k_cache, v_cache, new_k, new_v, block_tables, cache_lens, alibi_slopes=None, scale: float = 1.0, *, out=None,
                      pos_ids=None, sin_table=None, cos_table=None, rope_algo: int = RopeAlgo.GPT_NEOX):
    """One decode layer's cache update and attention behind one call (no reference counterpart: the
    reference's callers issue paged_caching and paged_attention).  new_k / new_v [num_seqs, num_kv_heads,
    head_size] are written to position cache_lens[i] - 1 of sequence i (the slot its block table names),
    then q attends over the cache_lens[i] positions.  Returns `out`; the caches are updated in place.

    With pos_ids [num_seqs], sin_table and cos_table [table_len, head_size / 2] the call also does the work
    of rope(q) and rope(new_k) first: the cache receives the rotated K row and the attention uses the rotated
    q (q and new_k themselves are left as they are)."""
    if pos_ids is not None:
        return _paged_decode_step_rope(q, k_cache, v_cache, new_k, new_v, block_tables, cache_lens, alibi_slopes, scale, out,
                                       pos_ids, sin_table, cos_table, rope_algo)
    dev = _require_cuda(q, k_cache, v_cache, new_k, new_v, block_tables, cache_lens, alibi_slopes, out)
    if out is None:
        out = torch.empty((*q.shape[:-1], v_cache.shape[3]), dtype=q.dtype, device=q.device)
    st = _state(dev)
    key = ("paged_decode_step", _meta(out), _meta(q), _meta(k_cache), _meta(v_cache), _meta(new_k), _meta(new_v),
           _meta(block_tables), _meta(cache_lens), _meta(alibi_slopes), float(scale))

    def make():
        tensors = [_desc(out), _desc(q), _desc(k_cache), _desc(v_cache), _desc(new_k), _desc(new_v), _desc(block_tables), _desc(cache_lens)]
        alibi = _desc(alibi_slopes) if alibi_slopes is not None else None
        desc = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedDecodeStepDescriptor(
            st["handle"], ctypes.byref(desc), *[t.descriptor for t in tensors],
            alibi.descriptor if alibi is not None else None, scale))
        size = ctypes.c_size_t(0)
        check_error(LIBINFINIOP.infiniopGetPagedDecodeStepWorkspaceSize(desc, ctypes.byref(size)))
        for t in tensors + ([alibi] if alibi is not None else []):
            t.destroy_desc()
        return {"desc": desc, "workspace": size.value, "destroy": LIBINFINIOP.infiniopDestroyPagedDecodeStepDescriptor}

    entry = _lookup(st, key, make)
    ws = _workspace(st, entry["workspace"], dev)
    with torch.cuda.device(dev):
        check_error(LIBINFINIOP.infiniopPagedDecodeStep(
            entry["desc"], ws.data_ptr() if ws is not None else None, entry["workspace"],
            out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), new_k.data_ptr(), new_v.data_ptr(),
            block_tables.data_ptr(), cache_lens.data_ptr(),
            alibi_slopes.data_ptr() if alibi_slopes is not None else None,
            torch.cuda.current_stream(dev).cuda_stream))
    return out


def _paged_decode_step_rope(q, k_cache, v_cache, new_k, new_v, block_tables, cache_lens, alibi_slopes, scale, out,
                            pos_ids, sin_table, cos_table, rope_algo):
    dev = _require_cuda(q, k_cache, v_cache, new_k, new_v, block_tables, cache_lens, alibi_slopes, out, pos_ids, sin_table, cos_table)
    if out is None:
        out = torch.empty((*q.shape[:-1], v_cache.shape[3]), dtype=q.dtype, device=q.device)
    st = _state(dev)
    key = ("paged_decode_step_rope", _meta(out), _meta(q), _meta(k_cache), _meta(v_cache), _meta(new_k), _meta(new_v),
           _meta(block_tables), _meta(cache_lens), _meta(alibi_slopes), _meta(pos_ids), _meta(sin_table), _meta(cos_table),
           int(rope_algo), float(scale))

    def make():
        tensors = [_desc(out), _desc(q), _desc(k_cache), _desc(v_cache), _desc(new_k), _desc(new_v), _desc(block_tables), _desc(cache_lens)]
        rope_tensors = [_desc(pos_ids), _desc(sin_table), _desc(cos_table)]
        alibi = _desc(alibi_slopes) if alibi_slopes is not None else None
        desc = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedDecodeStepRoPEDescriptor(
            st["handle"], ctypes.byref(desc), *[t.descriptor for t in tensors],
            alibi.descriptor if alibi is not None else None, *[t.descriptor for t in rope_tensors], int(rope_algo), scale))
        size = ctypes.c_size_t(0)
        check_error(LIBINFINIOP.infiniopGetPagedDecodeStepWorkspaceSize(desc, ctypes.byref(size)))
        for t in tensors + rope_tensors + ([alibi] if alibi is not None else []):
            t.destroy_desc()
        return {"desc": desc, "workspace": size.value, "destroy": LIBINFINIOP.infiniopDestroyPagedDecodeStepDescriptor}

    entry = _lookup(st, key, make)
    ws = _workspace(st, entry["workspace"], dev)
    with torch.cuda.device(dev):
        check_error(LIBINFINIOP.infiniopPagedDecodeStepRoPE(
            entry["desc"], ws.data_ptr() if ws is not None else None, entry["workspace"],
            out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), new_k.data_ptr(), new_v.data_ptr(),
            block_tables.data_ptr(), cache_lens.data_ptr(),
            alibi_slopes.data_ptr() if alibi_slopes is not None else None,
            pos_ids.data_ptr(), sin_table.data_ptr(), cos_table.data_ptr(),
            torch.cuda.current_stream(dev).cuda_stream))
    return out


def kv_caching(k_cache, v_cache, k, v, past_kv_lengths):
    """Appends k / v [batch, kv_heads, seq_len, hidden] to the contiguous caches [batch, kv_heads, max_seq_len, hidden]
    behind the past_kv_lengths[b] rows each sequence holds (the reference's infiniopKVCaching).  Returns (k_cache, v_cache)."""
    dev = _require_cuda(k_cache, v_cache, k, v, past_kv_lengths)
    st = _state(dev)
    key = ("kv_caching", _meta(k_cache), _meta(v_cache), _meta(k), _meta(v), _meta(past_kv_lengths))

    def make():
        tensors = [_desc(k_cache), _desc(v_cache), _desc(k), _desc(v), _desc(past_kv_lengths)]
        desc = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreateKVCachingDescriptor(
            st["handle"], ctypes.byref(desc), *[t.descriptor for t in tensors]))
        for t in tensors:
            t.destroy_desc()
        return {"desc": desc, "workspace": 0, "destroy": LIBINFINIOP.infiniopDestroyKVCachingDescriptor}

    entry = _lookup(st, key, make)
    with torch.cuda.device(dev):
        check_error(LIBINFINIOP.infiniopKVCaching(
            entry["desc"], None, 0, k_cache.data_ptr(), v_cache.data_ptr(), k.data_ptr(), v.data_ptr(),
            past_kv_lengths.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
    return (k_cache, v_cache)


def paged_caching(k_cache, v_cache, k, v, slot_mapping):
    """Scatters k/v rows [num_tokens, num_kv_heads, head_size] into the paged pools at
    slot_mapping (int64; negative = padding).  Returns (k_cache, v_cache)."""
    dev = _require_cuda(k_cache, v_cache, k, v, slot_mapping)
    st = _state(dev)
    key = ("paged_caching", _meta(k_cache), _meta(v_cache), _meta(k), _meta(v), _meta(slot_mapping))

    def make():
        tensors = [_desc(k_cache), _desc(v_cache), _desc(k), _desc(v), _desc(slot_mapping)]
        desc = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedCachingDescriptor(
            st["handle"], ctypes.byref(desc), *[t.descriptor for t in tensors]))
        for t in tensors:
            t.destroy_desc()
        return {"desc": desc, "workspace": 0, "destroy": LIBINFINIOP.infiniopDestroyPagedCachingDescriptor}

    entry = _lookup(st, key, make)
    with torch.cuda.device(dev):
        check_error(LIBINFINIOP.infiniopPagedCaching(
            entry["desc"], None, 0, k_cache.data_ptr(), v_cache.data_ptr(), k.data_ptr(), v.data_ptr(),
            slot_mapping.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
    return (k_cache, v_cache)
