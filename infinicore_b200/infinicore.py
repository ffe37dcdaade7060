"""The part of the reference's `infinicore` Python package that its paged-operator tests use
(test/infinicore/ops/paged_attention.py:211-215, test/infinicore/ops/paged_caching.py:212-220), over this
library's own pybind module `_infinicore_b200`:

    import infinicore_b200.infinicore as infinicore
    out = infinicore.paged_attention(q, k_cache, v_cache, block_tables, cache_lens, alibi_slopes=None, scale=s)
    infinicore.paged_caching(k_cache.permute([0, 2, 1, 3]), v_cache.permute([0, 2, 1, 3]), k, v, slot_mapping)
    infinicore.sync_stream()

Same function names, argument order, keyword names and return values as python/infinicore/ops/paged_attention.py:5-41
and python/infinicore/ops/paged_caching.py:5-22.  A Tensor wraps `_infinicore_b200.Tensor` the way the reference's
wraps `_infinicore.Tensor` (`._underlying`); it can be made from a torch CUDA tensor (`from_torch`, zero copy, the
torch tensor is kept alive) and turned back into one (`to_torch`).  The reference's allocator, tensor arithmetic,
printing and the rest of its ~180 operators are not here.
"""
from __future__ import annotations

import torch

from . import _infinicore_b200 as _C

DataType = _C.DataType
float16, bfloat16, float32, float64 = DataType.F16, DataType.BF16, DataType.F32, DataType.F64
int32, int64, uint8, bool_ = DataType.I32, DataType.I64, DataType.U8, DataType.BOOL

_FROM_TORCH = {torch.float16: float16, torch.bfloat16: bfloat16, torch.float32: float32, torch.float64: float64,
               torch.int32: int32, torch.int64: int64, torch.uint8: uint8, torch.bool: bool_}
_TO_TORCH = {v: k for k, v in _FROM_TORCH.items()}


class Tensor:
    """Device tensor as the operators see it: pointer, dtype, shape, element strides."""

    def __init__(self, underlying, keep_alive=None):
        self._underlying = underlying
        self._keep_alive = keep_alive  # whoever owns the memory of a view (a torch tensor)

    @property
    def shape(self):
        return list(self._underlying.shape)

    @property
    def dtype(self):
        return self._underlying.dtype

    def stride(self):
        return list(self._underlying.strides)

    def data_ptr(self):
        return self._underlying.data_ptr()

    def permute(self, dims):
        """A view with its dimensions reordered (no data moves), like the reference's Tensor.permute."""
        shape, strides = self.shape, self.stride()
        if sorted(dims) != list(range(len(shape))):
            raise ValueError(f"permute: {dims} is not a permutation of the {len(shape)} dimensions")
        view = _C.Tensor.from_blob(self.data_ptr(), [shape[d] for d in dims], [strides[d] for d in dims], self.dtype,
                                   self._underlying.device_index)
        return Tensor(view, keep_alive=self)

    def to_torch(self) -> torch.Tensor:
        """A torch tensor on the same memory (zero copy) for views made from torch; a copy for memory this
        package allocated."""
        base = self
        while isinstance(base._keep_alive, Tensor):
            base = base._keep_alive
        if isinstance(base._keep_alive, torch.Tensor):
            root = base._keep_alive
            offset = (self.data_ptr() - root.data_ptr()) // root.element_size()
            return torch.as_strided(root, self.shape, self.stride(), root.storage_offset() + offset)
        # memory from infinirtMalloc: copy out through a torch tensor of the same geometry
        dev = torch.device("cuda", self._underlying.device_index)
        out = torch.empty(self.shape, dtype=_TO_TORCH[self.dtype], device=dev)
        nbytes = out.numel() * out.element_size()
        if nbytes:
            import ctypes

            from .libinfiniop import LIBINFINIOP, check_error

            _C.sync_device()
            check_error(LIBINFINIOP.infinirtMemcpy(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(self.data_ptr()), nbytes, 3))  # device to device
        return out


def from_torch(t: torch.Tensor) -> Tensor:
    if not t.is_cuda:
        raise RuntimeError("infinicore_b200 runs on CUDA tensors only; there is no CPU path")
    view = _C.Tensor.from_blob(t.data_ptr(), list(t.shape), list(t.stride()), _FROM_TORCH[t.dtype], t.device.index or 0)
    return Tensor(view, keep_alive=t)


def paged_attention(q: Tensor, k_cache: Tensor, v_cache: Tensor, block_tables: Tensor, cache_lens: Tensor,
                    alibi_slopes: Tensor | None = None, scale: float = 1.0, *, out: Tensor | None = None):
    if out is None:
        return Tensor(_C.paged_attention(q._underlying, k_cache._underlying, v_cache._underlying, block_tables._underlying,
                                         cache_lens._underlying, alibi_slopes._underlying if alibi_slopes is not None else None, scale))
    _C.paged_attention_(out._underlying, q._underlying, k_cache._underlying, v_cache._underlying, block_tables._underlying,
                        cache_lens._underlying, alibi_slopes._underlying if alibi_slopes is not None else None, scale)
    return out


def paged_caching(k_cache: Tensor, v_cache: Tensor, k: Tensor, v: Tensor, slot_mapping: Tensor):
    _C.paged_caching_(k_cache._underlying, v_cache._underlying, k._underlying, v._underlying, slot_mapping._underlying)
    return (k_cache, v_cache)


def paged_attention_prefill(q: Tensor, k_cache: Tensor, v_cache: Tensor, block_tables: Tensor, total_kv_lens: Tensor,
                            cum_seqlens_q: Tensor, alibi_slopes: Tensor | None = None, scale: float = 1.0, *, out: Tensor):
    _C.paged_attention_prefill_(out._underlying, q._underlying, k_cache._underlying, v_cache._underlying, block_tables._underlying,
                                total_kv_lens._underlying, cum_seqlens_q._underlying,
                                alibi_slopes._underlying if alibi_slopes is not None else None, scale)
    return out


set_stream, get_stream, sync_stream, sync_device, set_device = _C.set_stream, _C.get_stream, _C.sync_stream, _C.sync_device, _C.set_device
kernel_status = _C.kernel_status
