"""Calls the two operators through the C ABI exactly as the reference's own tests do
(test/infiniop/paged_attention.py:202-251, test/infiniop/paged_caching.py:164-212): build
tensor descriptors, create the operator descriptor, query the workspace, destroy the tensor
descriptors BEFORE executing, execute on the NULL stream with a 0x01-filled workspace."""
from __future__ import annotations

import contextlib
import ctypes
import os

import torch

from infinicore_b200.libinfiniop import (
    LIBINFINIOP, InfiniDeviceEnum, InfiniDtype, TestTensor, TestWorkspace, check_error, create_handle,
    destroy_handle, infiniopOperatorDescriptor_t, to_infini_dtype,
)

_handle = None


def handle():
    global _handle
    if _handle is None:
        check_error(LIBINFINIOP.infinirtSetDevice(InfiniDeviceEnum.NVIDIA, 0))
        _handle = create_handle()
    return _handle


# Named variants of the decode path.  Every knob is read when the descriptor is created.
PATH_ENV = {
    None: {},
    "generic": {"INFINIOP_PAGED_DECODE_PATH": "generic"},
    "stream": {"INFINIOP_PAGED_DECODE_PATH": "stream"},
    # plan computed by the separate one-CTA kernel instead of inside the main kernel, plain launches
    "stream-plan-kernel": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_DECODE_EMBEDDED_PLAN": "0",
                           "INFINIOP_PAGED_DECODE_PDL": "0"},
    # other ring geometry: 3 warps per CTA, 4 slots
    "stream-3x4": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_DECODE_WARPS": "3", "INFINIOP_PAGED_DECODE_STAGES": "4"},
    # split units merged by the combine kernel instead of by the last worker to arrive
    "stream-combine": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_DECODE_MERGE_IN_KERNEL": "0"},
    # ranges cut into pieces, tail chunks claimed from the shared pool (merged in the kernel / by the combine kernel)
    "stream-pool": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_DECODE_CHUNKS": "4"},
    "stream-pool-combine": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_DECODE_CHUNKS": "3",
                            "INFINIOP_PAGED_DECODE_MIN_CHUNK": "2", "INFINIOP_PAGED_DECODE_MERGE_IN_KERNEL": "0"},
    # one copy per 64-element column chunk (the 4-D tensor maps; default at head 64 / 128) or one per tensor and
    # tile (the 5-D maps; default at key width 576)
    "stream-chunk-boxes": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_DECODE_ROW_BOXES": "0"},
    "stream-row-boxes": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_DECODE_ROW_BOXES": "1"},
    # block-table entries checked against the pool before use
    "stream-checked": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_CHECK_INDICES": "1"},
    "generic-checked": {"INFINIOP_PAGED_DECODE_PATH": "generic", "INFINIOP_PAGED_CHECK_INDICES": "1"},
    # the test of the bounded wait: worker 0 never issues its first copy and gives up after 20 ms
    "stream-withheld-copy": {"INFINIOP_PAGED_DECODE_PATH": "stream", "INFINIOP_PAGED_DECODE_TEST_WITHHOLD_COPY": "1",
                             "INFINIOP_PAGED_DECODE_WAIT_LIMIT_MS": "20"},
}


def kernel_status(stream=None):
    """infiniopGetKernelStatus on device 0: waits for the stream, returns the flag word and clears it."""
    flags = ctypes.c_uint32(0)
    check_error(LIBINFINIOP.infiniopGetKernelStatus(handle(), ctypes.c_void_p(stream), ctypes.byref(flags)))
    return flags.value


@contextlib.contextmanager
def environment(**values):
    """Environment variables for the duration of a descriptor creation (the library reads its knobs there)."""
    old = {k: os.environ.get(k) for k in values}
    os.environ.update({k: str(v) for k, v in values.items()})
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


@contextlib.contextmanager
def decode_path(path):
    """Sets the environment of one named path variant for the duration of a descriptor creation."""
    env = PATH_ENV[path]
    keys = {k for v in PATH_ENV.values() for k in v}
    old = {k: os.environ.get(k) for k in keys}
    for k in keys:
        os.environ.pop(k, None)
    os.environ.update(env)
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def _tt(t, dt=None):
    return TestTensor.from_torch(t, dt if dt is not None else to_infini_dtype(t.dtype), InfiniDeviceEnum.NVIDIA)


class AttentionOp:
    """One created paged-attention descriptor plus its workspace."""

    def __init__(self, out, q, k_cache, v_cache, block_tables, seq_lens, alibi, scale, path=None, index_dtype=None):
        tensors = [_tt(out), _tt(q), _tt(k_cache), _tt(v_cache), _tt(block_tables, index_dtype), _tt(seq_lens, index_dtype)]
        al = _tt(alibi) if alibi is not None else None
        self.desc = infiniopOperatorDescriptor_t()
        with decode_path(path):
            self.status = LIBINFINIOP.infiniopCreatePagedAttentionDescriptor(
                handle(), ctypes.byref(self.desc), *[t.descriptor for t in tensors],
                al.descriptor if al is not None else None, scale)
        for t in tensors + ([al] if al is not None else []):
            t.destroy_desc()
        self.workspace_size = 0
        self.workspace = None
        if self.status == 0:
            size = ctypes.c_size_t(0)
            check_error(LIBINFINIOP.infiniopGetPagedAttentionWorkspaceSize(self.desc, ctypes.byref(size)))
            self.workspace_size = size.value
            self.workspace = TestWorkspace(size.value, InfiniDeviceEnum.NVIDIA)

    def run(self, out, q, k_cache, v_cache, block_tables, seq_lens, alibi=None, stream=None, workspace_size=None):
        return LIBINFINIOP.infiniopPagedAttention(
            self.desc, self.workspace.data(), self.workspace_size if workspace_size is None else workspace_size,
            out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            block_tables.data_ptr(), seq_lens.data_ptr(), alibi.data_ptr() if alibi is not None else None, stream)

    def destroy(self):
        if self.status == 0 and self.desc:
            check_error(LIBINFINIOP.infiniopDestroyPagedAttentionDescriptor(self.desc))
            self.desc = None


class DecodeStepOp:
    """One created paged-decode-step descriptor (append + attention) plus its workspace."""

    def __init__(self, out, q, k_cache, v_cache, new_k, new_v, block_tables, seq_lens, alibi, scale, path=None, index_dtype=None):
        tensors = [_tt(out), _tt(q), _tt(k_cache), _tt(v_cache), _tt(new_k), _tt(new_v), _tt(block_tables, index_dtype),
                   _tt(seq_lens, index_dtype)]
        al = _tt(alibi) if alibi is not None else None
        self.desc = infiniopOperatorDescriptor_t()
        with decode_path(path):
            self.status = LIBINFINIOP.infiniopCreatePagedDecodeStepDescriptor(
                handle(), ctypes.byref(self.desc), *[t.descriptor for t in tensors],
                al.descriptor if al is not None else None, scale)
        for t in tensors + ([al] if al is not None else []):
            t.destroy_desc()
        self.workspace_size = 0
        self.workspace = None
        if self.status == 0:
            size = ctypes.c_size_t(0)
            check_error(LIBINFINIOP.infiniopGetPagedDecodeStepWorkspaceSize(self.desc, ctypes.byref(size)))
            self.workspace_size = size.value
            self.workspace = TestWorkspace(size.value, InfiniDeviceEnum.NVIDIA)

    def run(self, out, q, k_cache, v_cache, new_k, new_v, block_tables, seq_lens, alibi=None, stream=None):
        return LIBINFINIOP.infiniopPagedDecodeStep(
            self.desc, self.workspace.data(), self.workspace_size,
            out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), new_k.data_ptr(), new_v.data_ptr(),
            block_tables.data_ptr(), seq_lens.data_ptr(), alibi.data_ptr() if alibi is not None else None, stream)

    def destroy(self):
        if self.status == 0 and self.desc:
            check_error(LIBINFINIOP.infiniopDestroyPagedDecodeStepDescriptor(self.desc))
            self.desc = None


def paged_decode_step(q, k_cache, v_cache, new_k, new_v, block_tables, seq_lens, scale, alibi=None, path=None, out=None,
                      index_dtype=None):
    """Runs one append + decode call through the C ABI; returns `out` (synchronised); caches are updated in place."""
    if out is None:
        out = torch.zeros((*q.shape[:-1], v_cache.shape[3]), dtype=q.dtype, device=q.device)
    op = DecodeStepOp(out, q, k_cache, v_cache, new_k, new_v, block_tables, seq_lens, alibi, scale, path, index_dtype)
    check_error(op.status)
    try:
        check_error(op.run(out, q, k_cache, v_cache, new_k, new_v, block_tables, seq_lens, alibi))
        torch.cuda.synchronize()
    finally:
        op.destroy()
    return out


def kv_caching_create(k_cache, v_cache, k, v, past_kv_lengths, len_dtype=None):
    """Creates a KVCaching descriptor as reference test/infiniop/kv_caching.py:115-127 does; returns (status, descriptor)."""
    tensors = [_tt(k_cache), _tt(v_cache), _tt(k), _tt(v), _tt(past_kv_lengths, len_dtype)]
    desc = infiniopOperatorDescriptor_t()
    status = LIBINFINIOP.infiniopCreateKVCachingDescriptor(handle(), ctypes.byref(desc), *[t.descriptor for t in tensors])
    for t in tensors:
        t.destroy_desc()
    return status, desc


def kv_caching(k_cache, v_cache, k, v, past_kv_lengths, stream=None):
    """One infiniopKVCaching call through the C ABI; the caches are updated in place (synchronised)."""
    status, desc = kv_caching_create(k_cache, v_cache, k, v, past_kv_lengths)
    check_error(status)
    try:
        size = ctypes.c_size_t(1)
        check_error(LIBINFINIOP.infiniopGetKVCachingWorkspaceSize(desc, ctypes.byref(size)))
        assert size.value == 0
        check_error(LIBINFINIOP.infiniopKVCaching(desc, None, 0, k_cache.data_ptr(), v_cache.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                  past_kv_lengths.data_ptr(), stream))
        torch.cuda.synchronize()
    finally:
        check_error(LIBINFINIOP.infiniopDestroyKVCachingDescriptor(desc))


def rope_create(y, x, pos_ids, sin_table, cos_table, algo, pos_dtype=None):
    """Creates a RoPE descriptor as reference test/infiniop/rope.py:170-186 does; returns (status, descriptor)."""
    tensors = [_tt(y), _tt(x), _tt(pos_ids, pos_dtype), _tt(sin_table), _tt(cos_table)]
    desc = infiniopOperatorDescriptor_t()
    status = LIBINFINIOP.infiniopCreateRoPEDescriptor(handle(), ctypes.byref(desc), *[t.descriptor for t in tensors], int(algo))
    for t in tensors:
        t.destroy_desc()
    return status, desc


def rope(x, pos_ids, sin_table, cos_table, algo, y=None, pos_dtype=None):
    """One infiniopRoPE call through the C ABI on the NULL stream; returns y (x itself for the in-place form)."""
    if y is None:
        y = torch.zeros_like(x)
    status, desc = rope_create(y, x, pos_ids, sin_table, cos_table, algo, pos_dtype)
    check_error(status)
    try:
        size = ctypes.c_size_t(1)
        check_error(LIBINFINIOP.infiniopGetRoPEWorkspaceSize(desc, ctypes.byref(size)))
        assert size.value == 0
        check_error(LIBINFINIOP.infiniopRoPE(desc, None, 0, y.data_ptr(), x.data_ptr(), pos_ids.data_ptr(),
                                             sin_table.data_ptr(), cos_table.data_ptr(), None))
        torch.cuda.synchronize()
    finally:
        check_error(LIBINFINIOP.infiniopDestroyRoPEDescriptor(desc))
    return y


def paged_decode_step_rope(q, k_cache, v_cache, new_k, new_v, block_tables, seq_lens, scale, pos_ids, sin_table, cos_table, algo,
                           alibi=None, path=None, out=None, index_dtype=None, pos_dtype=None):
    """One rotate + append + decode call through the C ABI; returns `out` (synchronised); caches are updated in place."""
    if out is None:
        out = torch.zeros((*q.shape[:-1], v_cache.shape[3]), dtype=q.dtype, device=q.device)
    tensors = [_tt(out), _tt(q), _tt(k_cache), _tt(v_cache), _tt(new_k), _tt(new_v), _tt(block_tables, index_dtype),
               _tt(seq_lens, index_dtype)]
    rope_tensors = [_tt(pos_ids, pos_dtype), _tt(sin_table), _tt(cos_table)]
    al = _tt(alibi) if alibi is not None else None
    desc = infiniopOperatorDescriptor_t()
    with decode_path(path):
        status = LIBINFINIOP.infiniopCreatePagedDecodeStepRoPEDescriptor(
            handle(), ctypes.byref(desc), *[t.descriptor for t in tensors], al.descriptor if al is not None else None,
            *[t.descriptor for t in rope_tensors], int(algo), scale)
    for t in tensors + rope_tensors + ([al] if al is not None else []):
        t.destroy_desc()
    check_error(status)
    try:
        size = ctypes.c_size_t(0)
        check_error(LIBINFINIOP.infiniopGetPagedDecodeStepWorkspaceSize(desc, ctypes.byref(size)))
        workspace = TestWorkspace(size.value, InfiniDeviceEnum.NVIDIA)
        # the plain entry point refuses a descriptor of the RoPE form
        assert LIBINFINIOP.infiniopPagedDecodeStep(
            desc, workspace.data(), size.value, out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            new_k.data_ptr(), new_v.data_ptr(), block_tables.data_ptr(), seq_lens.data_ptr(), None, None) == 3
        check_error(LIBINFINIOP.infiniopPagedDecodeStepRoPE(
            desc, workspace.data(), size.value, out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            new_k.data_ptr(), new_v.data_ptr(), block_tables.data_ptr(), seq_lens.data_ptr(),
            alibi.data_ptr() if alibi is not None else None, pos_ids.data_ptr(), sin_table.data_ptr(), cos_table.data_ptr(), None))
        torch.cuda.synchronize()
        # the workspace ends with the rotated q and K rows; what precedes them (if anything) is the streaming kernel's
        r256 = lambda n: (n + 255) // 256 * 256
        rotated = r256(q.shape[0] * q.shape[1] * q.shape[2] * q.element_size()) + r256(new_k.numel() * new_k.element_size())
        assert size.value >= rotated
    finally:
        check_error(LIBINFINIOP.infiniopDestroyPagedDecodeStepDescriptor(desc))
    return out


def paged_attention(q, k_cache, v_cache, block_tables, seq_lens, scale, alibi=None, path=None, out=None,
                    index_dtype=None):
    """Runs one decode call through the C ABI; returns `out` (synchronised)."""
    if out is None:
        out = torch.zeros((*q.shape[:-1], v_cache.shape[3]), dtype=q.dtype, device=q.device)
    op = AttentionOp(out, q, k_cache, v_cache, block_tables, seq_lens, alibi, scale, path, index_dtype)
    check_error(op.status)
    try:
        check_error(op.run(out, q, k_cache, v_cache, block_tables, seq_lens, alibi))
        torch.cuda.synchronize()
    finally:
        op.destroy()
    return out


# Prefill variants: name -> environment read when the descriptor is created.  The tcgen05 kernel
# serves two q-heads of an even GQA group per CTA by default; "umma-q1" pins one q-head per CTA.
PREFILL_ENV = {
    None: {},
    "generic": {"INFINIOP_PAGED_PREFILL_PATH": "generic"},
    "tiles": {"INFINIOP_PAGED_PREFILL_PATH": "tiles"},
    "umma": {"INFINIOP_PAGED_PREFILL_PATH": "umma"},
    "umma-q1": {"INFINIOP_PAGED_PREFILL_PATH": "umma", "INFINIOP_PAGED_PREFILL_QTILES": "1"},
    "umma-q2-s3": {"INFINIOP_PAGED_PREFILL_PATH": "umma", "INFINIOP_PAGED_PREFILL_QTILES": "2", "INFINIOP_PAGED_PREFILL_STAGES": "3"},
    # every V copy from the second tile on held back 3 us: the P.V issuer falls behind the softmax warps
    "umma-late-v": {"INFINIOP_PAGED_PREFILL_PATH": "umma", "INFINIOP_PAGED_PREFILL_TEST_DELAY_V_US": "3"},
    "umma-late-v-k2": {"INFINIOP_PAGED_PREFILL_PATH": "umma", "INFINIOP_PAGED_PREFILL_TEST_DELAY_V_US": "3", "INFINIOP_PAGED_PREFILL_K_STAGES": "2"},
}
_PREFILL_KEYS = ("INFINIOP_PAGED_PREFILL_PATH", "INFINIOP_PAGED_PREFILL_QTILES", "INFINIOP_PAGED_PREFILL_STAGES", "INFINIOP_PAGED_PREFILL_K_STAGES",
                 "INFINIOP_PAGED_PREFILL_TEST_DELAY_V_US")


@contextlib.contextmanager
def prefill_path(path):
    """The INFINIOP_PAGED_PREFILL_* variables are read when the descriptor is created."""
    env = PREFILL_ENV[path] if path in PREFILL_ENV else {"INFINIOP_PAGED_PREFILL_PATH": path}
    old = {k: os.environ.get(k) for k in _PREFILL_KEYS}
    for k in _PREFILL_KEYS:
        os.environ.pop(k, None)
    os.environ.update(env)
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def create_prefill(out, q, k_cache, v_cache, block_tables, seq_lens, cum_q, alibi, scale, path=None, index_dtype=None):
    tensors = [_tt(out), _tt(q), _tt(k_cache), _tt(v_cache), _tt(block_tables, index_dtype), _tt(seq_lens, index_dtype),
               _tt(cum_q, index_dtype)]
    al = _tt(alibi) if alibi is not None else None
    desc = infiniopOperatorDescriptor_t()
    with prefill_path(path):
        status = LIBINFINIOP.infiniopCreatePagedAttentionPrefillDescriptor(
            handle(), ctypes.byref(desc), *[t.descriptor for t in tensors], al.descriptor if al is not None else None, scale)
    for t in tensors + ([al] if al is not None else []):
        t.destroy_desc()
    return status, desc


def paged_attention_prefill(q, k_cache, v_cache, block_tables, seq_lens, cum_q, scale, alibi=None, path=None, out=None,
                            index_dtype=None, stream=None):
    """Runs one prefill call through the C ABI (descriptors destroyed before execute); returns `out`."""
    if out is None:
        out = torch.zeros((*q.shape[:-1], v_cache.shape[3]), dtype=q.dtype, device=q.device)
    status, desc = create_prefill(out, q, k_cache, v_cache, block_tables, seq_lens, cum_q, alibi, scale, path, index_dtype)
    check_error(status)
    size = ctypes.c_size_t(99)
    check_error(LIBINFINIOP.infiniopGetPagedAttentionPrefillWorkspaceSize(desc, ctypes.byref(size)))
    ws = TestWorkspace(size.value, InfiniDeviceEnum.NVIDIA)
    try:
        check_error(LIBINFINIOP.infiniopPagedAttentionPrefill(
            desc, ws.data(), size.value, out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            block_tables.data_ptr(), seq_lens.data_ptr(), cum_q.data_ptr(), alibi.data_ptr() if alibi is not None else None, stream))
        torch.cuda.synchronize()
    finally:
        check_error(LIBINFINIOP.infiniopDestroyPagedAttentionPrefillDescriptor(desc))
    return out


def create_caching(k_cache, v_cache, k, v, slot_mapping, slot_dtype=None):
    tensors = [_tt(k_cache), _tt(v_cache), _tt(k), _tt(v), _tt(slot_mapping, slot_dtype)]
    desc = infiniopOperatorDescriptor_t()
    status = LIBINFINIOP.infiniopCreatePagedCachingDescriptor(handle(), ctypes.byref(desc), *[t.descriptor for t in tensors])
    for t in tensors:
        t.destroy_desc()
    return status, desc


def paged_caching(k_cache, v_cache, k, v, slot_mapping, stream=None):
    status, desc = create_caching(k_cache, v_cache, k, v, slot_mapping)
    check_error(status)
    size = ctypes.c_size_t(123)
    check_error(LIBINFINIOP.infiniopGetPagedCachingWorkspaceSize(desc, ctypes.byref(size)))
    assert size.value == 0
    try:
        check_error(LIBINFINIOP.infiniopPagedCaching(desc, None, 0, k_cache.data_ptr(), v_cache.data_ptr(),
                                                     k.data_ptr(), v.data_ptr(), slot_mapping.data_ptr(), stream))
        torch.cuda.synchronize()
    finally:
        check_error(LIBINFINIOP.infiniopDestroyPagedCachingDescriptor(desc))


def shutdown():
    global _handle
    if _handle is not None:
        destroy_handle(_handle)
        _handle = None
