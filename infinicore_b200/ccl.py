"""ctypes binding of libinfiniccl.so (the InfiniCCL C ABI over NCCL) for torch tensors.

Mirrors what a C caller of include/infiniccl.h does: one `Communicator` per device, collectives
issued on the caller's current CUDA stream.  Two ways to form a group, as in the reference
(include/infiniccl.h:24-37): `init_all(device_ids)` inside one process, or `unique_id()` on rank 0
+ `init_rank(nranks, token, rank)` on every rank of a one-process-per-GPU job (the token travels
by whatever the job already has - here a torch.distributed object broadcast).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char, c_int, c_size_t, c_void_p
from pathlib import Path

import torch

from .libinfiniop import InfiniDeviceEnum, check_error, to_infini_dtype

_PKG = Path(__file__).resolve().parent

SUM, PROD, MAX, MIN, AVG = 0, 1, 2, 3, 4
UNIQUE_ID_BYTES = 128

INFINICCL_SYMBOLS = [
    "infinicclCommInitAll", "infinicclGetUniqueId", "infinicclCommInitRank", "infinicclCommDestroy",
    "infinicclGroupStart", "infinicclGroupEnd", "infinicclAllReduce", "infinicclBroadcast",
    "infinicclSend", "infinicclRecv", "infinicclAllGather", "infinicclAllGatherV",
    "infinicclReduceScatter", "infinicclReduceScatterV",
]


class UniqueId(ctypes.Structure):
    _fields_ = [("internal", c_char * UNIQUE_ID_BYTES)]


def library_path() -> Path:
    dirs = []
    root = os.getenv("INFINI_ROOT")
    if root:
        dirs.append(Path(root) / "lib")
    dirs.append(_PKG / "lib")
    for d in dirs:
        if (d / "libinfiniccl.so").is_file():
            return d / "libinfiniccl.so"
    raise FileNotFoundError("libinfiniccl.so not found in " + ", ".join(map(str, dirs))
                            + "; build it with `python -m infinicore_b200.build`")


_LIB = None


def lib():
    """Loads libinfiniccl.so once (libinfinirt.so first: it is a dependency by soname)."""
    global _LIB
    if _LIB is None:
        path = library_path()
        ctypes.CDLL(str(path.parent / "libinfinirt.so"), mode=ctypes.RTLD_GLOBAL)
        l = ctypes.CDLL(str(path))
        l.infinicclCommInitAll.argtypes = [c_int, POINTER(c_void_p), c_int, POINTER(c_int)]
        l.infinicclGetUniqueId.argtypes = [POINTER(UniqueId)]
        l.infinicclCommInitRank.argtypes = [POINTER(c_void_p), c_int, UniqueId, c_int]
        l.infinicclCommDestroy.argtypes = [c_void_p]
        l.infinicclGroupStart.argtypes = [c_void_p]
        l.infinicclGroupEnd.argtypes = [c_void_p]
        l.infinicclAllReduce.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p]
        l.infinicclBroadcast.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p]
        l.infinicclSend.argtypes = [c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p]
        l.infinicclRecv.argtypes = [c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p]
        l.infinicclAllGather.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_void_p, c_void_p]
        l.infinicclAllGatherV.argtypes = [c_void_p, c_void_p, POINTER(c_size_t), c_int, c_int, c_void_p, c_void_p]
        l.infinicclReduceScatter.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p]
        l.infinicclReduceScatterV.argtypes = [c_void_p, c_void_p, POINTER(c_size_t), c_int, c_int, c_int, c_void_p, c_void_p]
        for name in INFINICCL_SYMBOLS:
            getattr(l, name).restype = c_int
        _LIB = l
    return _LIB


def _stream(device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _flat(t: torch.Tensor) -> torch.Tensor:
    if not t.is_contiguous():
        raise ValueError("collectives take contiguous tensors")
    return t


class Communicator:
    """One rank of a group; owns the C communicator until destroy()."""

    def __init__(self, handle: int, rank: int, world: int, device: int):
        self.handle, self.rank, self.world, self.device = c_void_p(handle), rank, world, device

    def destroy(self) -> None:
        if self.handle:
            check_error(lib().infinicclCommDestroy(self.handle))
            self.handle = c_void_p(None)

    def group_start(self) -> None:
        check_error(lib().infinicclGroupStart(self.handle))

    def group_end(self) -> None:
        check_error(lib().infinicclGroupEnd(self.handle))

    def all_reduce(self, send: torch.Tensor, recv: torch.Tensor, op: int = SUM) -> None:
        check_error(lib().infinicclAllReduce(_flat(send).data_ptr(), _flat(recv).data_ptr(), send.numel(), to_infini_dtype(send.dtype),
                                             op, self.handle, _stream(send.device)))

    def broadcast(self, send: torch.Tensor, recv: torch.Tensor, root: int) -> None:
        check_error(lib().infinicclBroadcast(_flat(send).data_ptr(), _flat(recv).data_ptr(), recv.numel(), to_infini_dtype(recv.dtype),
                                             root, self.handle, _stream(recv.device)))

    def send(self, t: torch.Tensor, peer: int) -> None:
        check_error(lib().infinicclSend(_flat(t).data_ptr(), t.numel(), to_infini_dtype(t.dtype), peer, self.handle, _stream(t.device)))

    def recv(self, t: torch.Tensor, peer: int) -> None:
        check_error(lib().infinicclRecv(_flat(t).data_ptr(), t.numel(), to_infini_dtype(t.dtype), peer, self.handle, _stream(t.device)))

    def all_gather(self, send: torch.Tensor, recv: torch.Tensor) -> None:
        """recv holds world * send.numel() elements, rank-major."""
        if recv.numel() != self.world * send.numel():
            raise ValueError("all_gather: recv must hold world * send elements")
        check_error(lib().infinicclAllGather(_flat(send).data_ptr(), _flat(recv).data_ptr(), send.numel(), to_infini_dtype(send.dtype),
                                             self.handle, _stream(send.device)))

    def all_gather_v(self, send: torch.Tensor, recv: torch.Tensor, counts) -> None:
        arr = (c_size_t * self.world)(*counts)
        check_error(lib().infinicclAllGatherV(_flat(send).data_ptr(), _flat(recv).data_ptr(), arr, self.world, to_infini_dtype(send.dtype),
                                              self.handle, _stream(send.device)))

    def reduce_scatter(self, send: torch.Tensor, recv: torch.Tensor, op: int = SUM) -> None:
        if send.numel() != self.world * recv.numel():
            raise ValueError("reduce_scatter: send must hold world * recv elements")
        check_error(lib().infinicclReduceScatter(_flat(send).data_ptr(), _flat(recv).data_ptr(), recv.numel(), to_infini_dtype(send.dtype),
                                                 op, self.handle, _stream(send.device)))

    def reduce_scatter_v(self, send: torch.Tensor, recv: torch.Tensor, counts, op: int = SUM) -> None:
        arr = (c_size_t * self.world)(*counts)
        check_error(lib().infinicclReduceScatterV(_flat(send).data_ptr(), _flat(recv).data_ptr(), arr, self.world,
                                                  to_infini_dtype(send.dtype), op, self.handle, _stream(send.device)))


def init_all(device_ids):
    """One process driving several devices: communicator i is rank i on device_ids[i]."""
    n = len(device_ids)
    comms = (c_void_p * n)()
    ids = (c_int * n)(*device_ids)
    check_error(lib().infinicclCommInitAll(InfiniDeviceEnum.NVIDIA, comms, n, ids))
    return [Communicator(comms[i], i, n, device_ids[i]) for i in range(n)]


def unique_id() -> bytes:
    uid = UniqueId()
    check_error(lib().infinicclGetUniqueId(ctypes.byref(uid)))
    return ctypes.string_at(ctypes.addressof(uid), UNIQUE_ID_BYTES)


def init_rank(nranks: int, token: bytes, rank: int) -> Communicator:
    """Joins the group named by `token` on the calling thread's current device."""
    uid = UniqueId()
    ctypes.memmove(ctypes.addressof(uid), token, UNIQUE_ID_BYTES)
    comm = c_void_p()
    check_error(lib().infinicclCommInitRank(ctypes.byref(comm), nranks, uid, rank))
    return Communicator(comm.value, rank, nranks, torch.cuda.current_device())


def init_from_process_group(group=None) -> Communicator:
    """A communicator spanning a torch.distributed group: rank 0 makes the token, a
    broadcast of a Python object carries it.  The current CUDA device must be set."""
    import torch.distributed as dist

    from .libinfiniop import LIBINFINIOP

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    check_error(LIBINFINIOP.infinirtSetDevice(InfiniDeviceEnum.NVIDIA, torch.cuda.current_device()))
    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    return init_rank(world, box[0], rank)
