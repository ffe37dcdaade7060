"""ctypes binding of libinfiniop / libinfinirt, shaped like the reference's test harness.

Mirrors reference test/infiniop/libinfiniop/{liboperators.py,structs.py,datatypes.py,devices.py,
utils.py}: the same names (LIBINFINIOP, InfiniDtype, InfiniDeviceEnum, TestTensor,
TestWorkspace, check_error, create_handle, ...) with the same meaning, restricted to the two
paged operators - the reference loader binds 89 operators and fails on the first missing symbol
(test/infiniop/libinfiniop/op_register.py:19-30); this one binds what this library exports.

The libraries are looked up in $INFINI_ROOT/lib first (the reference's convention) and then in
infinicore_b200/lib (the in-tree build).  There is no fallback: if they are missing or do not
load, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_void_p
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent


class InfiniDtype:
    INVALID, BYTE, BOOL, I8, I16, I32, I64, U8, U16, U32, U64, F8, F16, F32, F64, C16, C32, C64, C128, BF16 = range(20)


InfiniDtypeNames = {v: k for k, v in vars(InfiniDtype).items() if not k.startswith("_")}


class InfiniDeviceEnum:
    CPU, NVIDIA, CAMBRICON, ASCEND, METAX, MOORE, ILUVATAR, KUNLUN, HYGON, QY, ALI = range(11)


InfiniDeviceNames = {v: k for k, v in vars(InfiniDeviceEnum).items() if not k.startswith("_")}

torch_device_map = {InfiniDeviceEnum.CPU: "cpu", InfiniDeviceEnum.NVIDIA: "cuda"}

STATUS_NAMES = {
    0: "SUCCESS", 1: "INTERNAL_ERROR", 2: "NOT_IMPLEMENTED", 3: "BAD_PARAM", 4: "NULL_POINTER",
    5: "DEVICE_TYPE_NOT_SUPPORTED", 6: "DEVICE_NOT_FOUND", 7: "DEVICE_NOT_INITIALIZED",
    8: "DEVICE_ARCHITECTURE_NOT_SUPPORTED", 10: "BAD_TENSOR_DTYPE", 11: "BAD_TENSOR_SHAPE",
    12: "BAD_TENSOR_STRIDES", 13: "INSUFFICIENT_WORKSPACE",
}


class InfiniStatusError(RuntimeError):
    def __init__(self, status: int):
        self.status = status
        super().__init__(f"infiniop call failed: status {status} ({STATUS_NAMES.get(status, '?')})")


def check_error(status: int) -> None:
    if status != 0:
        raise InfiniStatusError(status)


class TensorDescriptor(Structure):
    _fields_ = []


infiniopTensorDescriptor_t = POINTER(TensorDescriptor)


class Handle(Structure):
    _fields_ = [("device", c_int), ("device_id", c_int)]


infiniopHandle_t = POINTER(Handle)


class OpDescriptor(Structure):
    _fields_ = [("device", c_int), ("device_id", c_int)]


infiniopOperatorDescriptor_t = POINTER(OpDescriptor)

# every extern "C" symbol declared in include/*.h, by library
INFINIOP_SYMBOLS = [
    "infiniopCreateHandle", "infiniopDestroyHandle",
    "infiniopCreateTensorDescriptor", "infiniopDestroyTensorDescriptor",
    "infiniopGetDescriptorDeviceType", "infiniopGetDescriptorDeviceId",
    "infiniopCreatePagedAttentionDescriptor", "infiniopGetPagedAttentionWorkspaceSize",
    "infiniopPagedAttention", "infiniopPagedAttentionStaticWorkspace", "infiniopPagedAttentionMultiOut",
    "infiniopDestroyPagedAttentionDescriptor",
    "infiniopCreatePagedAttentionPrefillDescriptor", "infiniopGetPagedAttentionPrefillWorkspaceSize",
    "infiniopPagedAttentionPrefill", "infiniopDestroyPagedAttentionPrefillDescriptor",
    "infiniopCreatePagedCachingDescriptor", "infiniopGetPagedCachingWorkspaceSize",
    "infiniopPagedCaching", "infiniopDestroyPagedCachingDescriptor",
    "infiniopCreatePagedDecodeStepDescriptor", "infiniopGetPagedDecodeStepWorkspaceSize",
    "infiniopPagedDecodeStep", "infiniopDestroyPagedDecodeStepDescriptor",
    "infiniopCreatePagedDecodeStepRoPEDescriptor", "infiniopPagedDecodeStepRoPE",
    "infiniopCreateRoPEDescriptor", "infiniopGetRoPEWorkspaceSize", "infiniopRoPE", "infiniopDestroyRoPEDescriptor",
    "infiniopCreateKVCachingDescriptor", "infiniopGetKVCachingWorkspaceSize", "infiniopKVCaching",
    "infiniopDestroyKVCachingDescriptor",
    "infiniopGetKernelStatus",
]
INFINIRT_SYMBOLS = [
    "infinirtInit", "infinirtGetAllDeviceCount", "infinirtGetDeviceCount", "infinirtSetDevice",
    "infinirtGetDevice", "infinirtGetMemInfo", "infinirtGetDeviceResourceSnapshot", "infinirtDeviceSynchronize",
    "infinirtStreamCreate", "infinirtStreamDestroy", "infinirtStreamSynchronize", "infinirtStreamWaitEvent",
    "infinirtEventCreate", "infinirtEventCreateWithFlags", "infinirtEventRecord", "infinirtEventQuery",
    "infinirtEventSynchronize", "infinirtEventDestroy", "infinirtEventElapsedTime",
    "infinirtMalloc", "infinirtMallocHost", "infinirtFree", "infinirtFreeHost",
    "infinirtMemcpy", "infinirtMemcpyAsync", "infinirtMallocAsync", "infinirtFreeAsync",
    "infinirtMemset", "infinirtMemsetAsync",
    "infinirtStreamBeginCapture", "infinirtStreamEndCapture", "infinirtGraphDestroy",
    "infinirtGraphInstantiate", "infinirtGraphExecDestroy", "infinirtGraphLuanch",
    "infinirtCommunicationBegin", "infinirtCommunicationEnd",
]


def library_paths():
    """(libinfinirt.so, libinfiniop.so) - $INFINI_ROOT/lib wins over the in-tree build."""
    dirs = []
    root = os.getenv("INFINI_ROOT")
    if root:
        dirs.append(Path(root) / "lib")
    dirs.append(_PKG / "lib")
    for d in dirs:
        rt, op = d / "libinfinirt.so", d / "libinfiniop.so"
        if rt.is_file() and op.is_file():
            return rt, op
    raise FileNotFoundError(
        "libinfinirt.so / libinfiniop.so not found in " + ", ".join(map(str, dirs))
        + "; build them with `python -m infinicore_b200.build` (there is no non-CUDA fallback)"
    )


class InfiniLib:
    def __init__(self, librt, libop):
        self.librt = librt
        self.libop = libop

    def __getattr__(self, name):
        for lib in (self.libop, self.librt):
            if hasattr(lib, name):
                return getattr(lib, name)
        raise AttributeError(f"Attribute {name} not found in library")


def _bind(lib: InfiniLib) -> None:
    op, rt = lib.libop, lib.librt
    op.infiniopCreateTensorDescriptor.argtypes = [POINTER(infiniopTensorDescriptor_t), c_uint64, POINTER(c_uint64), POINTER(c_int64), c_int]
    op.infiniopCreateTensorDescriptor.restype = c_int
    op.infiniopDestroyTensorDescriptor.argtypes = [infiniopTensorDescriptor_t]
    op.infiniopDestroyTensorDescriptor.restype = c_int
    op.infiniopCreateHandle.argtypes = [POINTER(infiniopHandle_t)]
    op.infiniopCreateHandle.restype = c_int
    op.infiniopDestroyHandle.argtypes = [infiniopHandle_t]
    op.infiniopDestroyHandle.restype = c_int
    op.infiniopGetDescriptorDeviceType.argtypes = [infiniopOperatorDescriptor_t, POINTER(c_int)]
    op.infiniopGetDescriptorDeviceType.restype = c_int
    op.infiniopGetDescriptorDeviceId.argtypes = [infiniopOperatorDescriptor_t, POINTER(c_int)]
    op.infiniopGetDescriptorDeviceId.restype = c_int

    # reference test/infiniop/libinfiniop/op_register.py:2188-2229
    op.infiniopCreatePagedAttentionDescriptor.restype = c_int32
    op.infiniopCreatePagedAttentionDescriptor.argtypes = [
        infiniopHandle_t, POINTER(infiniopOperatorDescriptor_t),
        infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
        infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
        c_void_p, c_float,
    ]
    op.infiniopGetPagedAttentionWorkspaceSize.restype = c_int32
    op.infiniopGetPagedAttentionWorkspaceSize.argtypes = [infiniopOperatorDescriptor_t, POINTER(c_size_t)]
    op.infiniopPagedAttention.restype = c_int32
    op.infiniopPagedAttention.argtypes = [
        infiniopOperatorDescriptor_t, c_void_p, c_size_t,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
    ]
    # No reference counterpart: same call without workspace arguments (scratch lives inside the
    # library).  Bound only where present, so this binding can also drive a build of the reference's
    # own library (which the parity tests do through $INFINI_ROOT).
    if hasattr(op, "infiniopPagedAttentionStaticWorkspace"):
        op.infiniopPagedAttentionStaticWorkspace.restype = c_int32
        op.infiniopPagedAttentionStaticWorkspace.argtypes = [
            infiniopOperatorDescriptor_t,
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        ]
    # No reference counterpart: every output row stored to several buffers (outs[0] the ordinary one).
    if hasattr(op, "infiniopPagedAttentionMultiOut"):
        op.infiniopPagedAttentionMultiOut.restype = c_int32
        op.infiniopPagedAttentionMultiOut.argtypes = [
            infiniopOperatorDescriptor_t, c_void_p, c_size_t, POINTER(c_void_p), c_size_t,
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        ]
    op.infiniopDestroyPagedAttentionDescriptor.restype = c_int32
    op.infiniopDestroyPagedAttentionDescriptor.argtypes = [infiniopOperatorDescriptor_t]
    # No reference counterpart: the device's word of kernel status flags, read and cleared.
    if hasattr(op, "infiniopGetKernelStatus"):
        op.infiniopGetKernelStatus.restype = c_int32
        op.infiniopGetKernelStatus.argtypes = [infiniopHandle_t, c_void_p, POINTER(c_uint32)]

    # reference test/infiniop/libinfiniop/op_register.py:2272-2320
    if hasattr(op, "infiniopCreatePagedAttentionPrefillDescriptor"):
        op.infiniopCreatePagedAttentionPrefillDescriptor.restype = c_int32
        op.infiniopCreatePagedAttentionPrefillDescriptor.argtypes = [
            infiniopHandle_t, POINTER(infiniopOperatorDescriptor_t),
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, c_void_p, c_float,
        ]
        op.infiniopGetPagedAttentionPrefillWorkspaceSize.restype = c_int32
        op.infiniopGetPagedAttentionPrefillWorkspaceSize.argtypes = [infiniopOperatorDescriptor_t, POINTER(c_size_t)]
        op.infiniopPagedAttentionPrefill.restype = c_int32
        op.infiniopPagedAttentionPrefill.argtypes = [
            infiniopOperatorDescriptor_t, c_void_p, c_size_t,
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        ]
        op.infiniopDestroyPagedAttentionPrefillDescriptor.restype = c_int32
        op.infiniopDestroyPagedAttentionPrefillDescriptor.argtypes = [infiniopOperatorDescriptor_t]

    # No reference counterpart: caching of the newest row + decode attention behind one call.
    if hasattr(op, "infiniopCreatePagedDecodeStepDescriptor"):
        op.infiniopCreatePagedDecodeStepDescriptor.restype = c_int32
        op.infiniopCreatePagedDecodeStepDescriptor.argtypes = [
            infiniopHandle_t, POINTER(infiniopOperatorDescriptor_t),
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
            c_void_p, c_float,
        ]
        op.infiniopGetPagedDecodeStepWorkspaceSize.restype = c_int32
        op.infiniopGetPagedDecodeStepWorkspaceSize.argtypes = [infiniopOperatorDescriptor_t, POINTER(c_size_t)]
        op.infiniopPagedDecodeStep.restype = c_int32
        op.infiniopPagedDecodeStep.argtypes = [
            infiniopOperatorDescriptor_t, c_void_p, c_size_t,
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        ]
        op.infiniopDestroyPagedDecodeStepDescriptor.restype = c_int32
        op.infiniopDestroyPagedDecodeStepDescriptor.argtypes = [infiniopOperatorDescriptor_t]

    # The same with the rotary embedding of q and of the new K row in front.
    if hasattr(op, "infiniopCreatePagedDecodeStepRoPEDescriptor"):
        op.infiniopCreatePagedDecodeStepRoPEDescriptor.restype = c_int32
        op.infiniopCreatePagedDecodeStepRoPEDescriptor.argtypes = [
            infiniopHandle_t, POINTER(infiniopOperatorDescriptor_t),
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
            c_void_p, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, c_int32, c_float,
        ]
        op.infiniopPagedDecodeStepRoPE.restype = c_int32
        op.infiniopPagedDecodeStepRoPE.argtypes = [
            infiniopOperatorDescriptor_t, c_void_p, c_size_t,
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
            c_void_p, c_void_p, c_void_p, c_void_p,
        ]

    # the signatures of reference include/infiniop/ops/rope.h:16-39
    if hasattr(op, "infiniopCreateRoPEDescriptor"):
        op.infiniopCreateRoPEDescriptor.restype = c_int32
        op.infiniopCreateRoPEDescriptor.argtypes = [
            infiniopHandle_t, POINTER(infiniopOperatorDescriptor_t),
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, c_int32,
        ]
        op.infiniopGetRoPEWorkspaceSize.restype = c_int32
        op.infiniopGetRoPEWorkspaceSize.argtypes = [infiniopOperatorDescriptor_t, POINTER(c_size_t)]
        op.infiniopRoPE.restype = c_int32
        op.infiniopRoPE.argtypes = [
            infiniopOperatorDescriptor_t, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        ]
        op.infiniopDestroyRoPEDescriptor.restype = c_int32
        op.infiniopDestroyRoPEDescriptor.argtypes = [infiniopOperatorDescriptor_t]

    # the signatures of reference include/infiniop/ops/kv_caching.h:8-29
    if hasattr(op, "infiniopCreateKVCachingDescriptor"):
        op.infiniopCreateKVCachingDescriptor.restype = c_int32
        op.infiniopCreateKVCachingDescriptor.argtypes = [
            infiniopHandle_t, POINTER(infiniopOperatorDescriptor_t),
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
            infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
        ]
        op.infiniopGetKVCachingWorkspaceSize.restype = c_int32
        op.infiniopGetKVCachingWorkspaceSize.argtypes = [infiniopOperatorDescriptor_t, POINTER(c_size_t)]
        op.infiniopKVCaching.restype = c_int32
        op.infiniopKVCaching.argtypes = [
            infiniopOperatorDescriptor_t, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        ]
        op.infiniopDestroyKVCachingDescriptor.restype = c_int32
        op.infiniopDestroyKVCachingDescriptor.argtypes = [infiniopOperatorDescriptor_t]

    # reference test/infiniop/libinfiniop/op_register.py:2231-2269
    op.infiniopCreatePagedCachingDescriptor.restype = c_int32
    op.infiniopCreatePagedCachingDescriptor.argtypes = [
        infiniopHandle_t, POINTER(infiniopOperatorDescriptor_t),
        infiniopTensorDescriptor_t, infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
        infiniopTensorDescriptor_t, infiniopTensorDescriptor_t,
    ]
    op.infiniopGetPagedCachingWorkspaceSize.restype = c_int32
    op.infiniopGetPagedCachingWorkspaceSize.argtypes = [infiniopOperatorDescriptor_t, POINTER(c_size_t)]
    op.infiniopPagedCaching.restype = c_int32
    op.infiniopPagedCaching.argtypes = [
        infiniopOperatorDescriptor_t, c_void_p, c_size_t,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
    ]
    op.infiniopDestroyPagedCachingDescriptor.restype = c_int32
    op.infiniopDestroyPagedCachingDescriptor.argtypes = [infiniopOperatorDescriptor_t]

    rt.infinirtSetDevice.argtypes = [c_int, c_int]
    rt.infinirtSetDevice.restype = c_int
    rt.infinirtGetDevice.argtypes = [POINTER(c_int), POINTER(c_int)]
    rt.infinirtGetDevice.restype = c_int
    rt.infinirtGetDeviceCount.argtypes = [c_int, POINTER(c_int)]
    rt.infinirtGetDeviceCount.restype = c_int
    rt.infinirtDeviceSynchronize.argtypes = []
    rt.infinirtDeviceSynchronize.restype = c_int
    for name in ("infinirtStreamCreate", "infinirtEventCreate"):
        getattr(rt, name).argtypes = [POINTER(c_void_p)]
        getattr(rt, name).restype = c_int
    for name in ("infinirtStreamDestroy", "infinirtStreamSynchronize", "infinirtEventSynchronize", "infinirtEventDestroy"):
        getattr(rt, name).argtypes = [c_void_p]
        getattr(rt, name).restype = c_int
    rt.infinirtEventRecord.argtypes = [c_void_p, c_void_p]
    rt.infinirtEventRecord.restype = c_int
    rt.infinirtEventElapsedTime.argtypes = [POINTER(c_float), c_void_p, c_void_p]
    rt.infinirtEventElapsedTime.restype = c_int
    rt.infinirtMalloc.argtypes = [POINTER(c_void_p), c_size_t]
    rt.infinirtMalloc.restype = c_int
    rt.infinirtMallocHost.argtypes = [POINTER(c_void_p), c_size_t]
    rt.infinirtMallocHost.restype = c_int
    rt.infinirtFree.argtypes = [c_void_p]
    rt.infinirtFree.restype = c_int
    rt.infinirtFreeHost.argtypes = [c_void_p]
    rt.infinirtFreeHost.restype = c_int
    rt.infinirtMemcpy.argtypes = [c_void_p, c_void_p, c_size_t, c_int]
    rt.infinirtMemcpy.restype = c_int
    rt.infinirtMemcpyAsync.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_void_p]
    rt.infinirtMemcpyAsync.restype = c_int
    rt.infinirtStreamBeginCapture.argtypes = [c_void_p, c_int]
    rt.infinirtStreamBeginCapture.restype = c_int
    rt.infinirtStreamEndCapture.argtypes = [c_void_p, POINTER(c_void_p)]
    rt.infinirtStreamEndCapture.restype = c_int
    rt.infinirtGraphInstantiate.argtypes = [POINTER(c_void_p), c_void_p, c_void_p, c_void_p, c_size_t]
    rt.infinirtGraphInstantiate.restype = c_int
    rt.infinirtGraphLuanch.argtypes = [c_void_p, c_void_p]
    rt.infinirtGraphLuanch.restype = c_int
    rt.infinirtGraphDestroy.argtypes = [c_void_p]
    rt.infinirtGraphDestroy.restype = c_int
    rt.infinirtGraphExecDestroy.argtypes = [c_void_p]
    rt.infinirtGraphExecDestroy.restype = c_int


def open_lib() -> InfiniLib:
    rt_path, op_path = library_paths()
    librt = ctypes.CDLL(str(rt_path), mode=ctypes.RTLD_GLOBAL)
    libop = ctypes.CDLL(str(op_path))
    lib = InfiniLib(librt, libop)
    _bind(lib)
    return lib


LIBINFINIOP = open_lib()


# ---- tensors -----------------------------------------------------------------------------

_TORCH_DTYPES = {
    InfiniDtype.F16: torch.float16, InfiniDtype.BF16: torch.bfloat16, InfiniDtype.F32: torch.float32,
    InfiniDtype.F64: torch.float64, InfiniDtype.I8: torch.int8, InfiniDtype.I16: torch.int16,
    InfiniDtype.I32: torch.int32, InfiniDtype.I64: torch.int64, InfiniDtype.U8: torch.uint8,
    InfiniDtype.U32: torch.int32,  # torch has no first-class uint32 storage ops; bits are what travels
    InfiniDtype.BOOL: torch.bool,
}


def to_torch_dtype(dt: int):
    return _TORCH_DTYPES[dt]


def to_infini_dtype(dt: torch.dtype) -> int:
    for k, v in _TORCH_DTYPES.items():
        if v == dt and k != InfiniDtype.U32:
            return k
    raise ValueError(f"unsupported torch dtype {dt}")


class CTensor:
    """Owns one infiniopTensorDescriptor_t (reference test/infiniop/libinfiniop/utils.py:16-43)."""

    def __init__(self, dt: int, shape, strides=None):
        self.ndim = len(shape)
        self.c_shape = (c_uint64 * self.ndim)(*shape)
        self.c_strides = (c_int64 * self.ndim)(*strides) if strides is not None else None
        self.dt = dt
        self.descriptor = infiniopTensorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreateTensorDescriptor(
            ctypes.byref(self.descriptor), self.ndim, self.c_shape, self.c_strides, dt))

    def destroy_desc(self):
        if self.descriptor is not None:
            LIBINFINIOP.infiniopDestroyTensorDescriptor(self.descriptor)
            self.descriptor = None


class TestTensor(CTensor):
    """A torch tensor plus its descriptor.  `from_torch` wraps an existing tensor (keeping its
    strides, so permuted views describe themselves), the constructor makes a fresh one
    (mode "random" is U(0,1) like the reference's, "zeros", "ones")."""

    __test__ = False  # not a pytest class

    def __init__(self, shape, strides, dt: int, device: int, mode="random", set_tensor=None):
        self.device = device
        dev = torch_device_map[device]
        if mode == "manual":
            assert set_tensor is not None
            self._torch_tensor = set_tensor.to(dev)
            shape = list(self._torch_tensor.shape)
            strides = list(self._torch_tensor.stride())
        elif mode == "random":
            self._torch_tensor = torch.rand(shape, dtype=to_torch_dtype(dt), device=dev)
        elif mode == "zeros":
            self._torch_tensor = torch.zeros(shape, dtype=to_torch_dtype(dt), device=dev)
        elif mode == "ones":
            self._torch_tensor = torch.ones(shape, dtype=to_torch_dtype(dt), device=dev)
        else:
            raise ValueError("Unsupported mode")
        self.shape = list(shape)
        self.strides = strides
        super().__init__(dt, shape, strides)

    @staticmethod
    def from_torch(torch_tensor, dt: int, device: int):
        return TestTensor(None, None, dt, device, mode="manual", set_tensor=torch_tensor)

    def torch_tensor(self):
        return self._torch_tensor

    def actual_tensor(self):
        return self._torch_tensor

    def data(self):
        return self._torch_tensor.data_ptr()


class TestWorkspace:
    """Caller-owned scratch, deliberately filled with 0x01 bytes as the reference's is
    (test/infiniop/libinfiniop/utils.py:292-297): kernels must not assume zeroed memory."""

    __test__ = False

    def __init__(self, size: int, device: int):
        self._size = size
        self.tensor = None
        if size:
            self.tensor = torch.ones(size, dtype=torch.uint8, device=torch_device_map[device])

    def data(self):
        return self.tensor.data_ptr() if self.tensor is not None else None

    def size(self):
        return self._size


def create_handle():
    handle = infiniopHandle_t()
    check_error(LIBINFINIOP.infiniopCreateHandle(ctypes.byref(handle)))
    return handle


def destroy_handle(handle):
    check_error(LIBINFINIOP.infiniopDestroyHandle(handle))
