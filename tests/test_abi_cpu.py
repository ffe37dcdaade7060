"""CPU-side checks of the C-ABI libraries: they load, export every symbol the public headers
declare, and the host-only entry points behave (no compute call is made here)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = {}
    for header in sorted((ROOT / "include").rglob("*.h")):
        for m in re.finditer(r"__INFINI_C\s+__export\s+infiniStatus_t\s+(\w+)\s*\(", header.read_text()):
            names[m.group(1)] = header.name
    return names


def test_headers_declare_the_expected_surface():
    names = declared_symbols()
    for must in ("infiniopCreatePagedAttentionDescriptor", "infiniopGetPagedAttentionWorkspaceSize",
                 "infiniopPagedAttention", "infiniopDestroyPagedAttentionDescriptor",
                 "infiniopCreatePagedCachingDescriptor", "infiniopGetPagedCachingWorkspaceSize",
                 "infiniopPagedCaching", "infiniopDestroyPagedCachingDescriptor",
                 "infiniopCreateHandle", "infiniopCreateTensorDescriptor", "infinirtSetDevice", "infinirtGetDevice"):
        assert must in names


def test_libraries_load_and_export_every_declared_symbol():
    from infinicore_b200 import libinfiniop as L

    rt_path, op_path = L.library_paths()
    from infinicore_b200 import ccl

    rt = ctypes.CDLL(str(rt_path), mode=ctypes.RTLD_GLOBAL)
    op = ctypes.CDLL(str(op_path))
    cc = ctypes.CDLL(str(ccl.library_path()))
    for name, header in declared_symbols().items():
        lib = rt if name.startswith("infinirt") else cc if name.startswith("infiniccl") else op
        assert hasattr(lib, name), f"{name} (declared in {header}) is not exported"
    # and the bindings' own lists are the same set
    assert set(L.INFINIOP_SYMBOLS) | set(L.INFINIRT_SYMBOLS) | set(ccl.INFINICCL_SYMBOLS) == set(declared_symbols())


def test_infiniccl_argument_checks_need_no_device():
    """Host-side refusals of libinfiniccl.so (reference src/infiniccl/infiniccl.cc: NULL checks first)."""
    from infinicore_b200 import ccl

    l = ccl.lib()
    assert l.infinicclGetUniqueId(None) == 4           # INFINI_STATUS_NULL_POINTER
    assert l.infinicclCommInitRank(None, 2, ccl.UniqueId(), 0) == 4
    assert l.infinicclCommDestroy(None) == 0            # NULL communicator: nothing to do
    assert l.infinicclGroupStart(None) == 4
    assert l.infinicclCommInitAll(0, None, 1, None) == 5  # CPU device type: not supported


def test_tensor_descriptor_round_trip_needs_no_device():
    from infinicore_b200.libinfiniop import CTensor, InfiniDtype

    t = CTensor(InfiniDtype.BF16, [4, 8, 128], None)
    assert bool(t.descriptor)
    t.destroy_desc()
    t = CTensor(InfiniDtype.F16, [16, 2, 16, 64], [2048, 64, 128, 1])
    t.destroy_desc()


def test_thread_local_device_defaults_to_cpu_and_handle_creation_is_refused():
    import threading

    from infinicore_b200.libinfiniop import LIBINFINIOP, InfiniDeviceEnum, infiniopHandle_t

    seen = {}

    def probe():
        dev, idx = ctypes.c_int(-1), ctypes.c_int(-1)
        seen["get"] = LIBINFINIOP.infinirtGetDevice(ctypes.byref(dev), ctypes.byref(idx))
        seen["dev"] = dev.value
        h = infiniopHandle_t()
        seen["create"] = LIBINFINIOP.infiniopCreateHandle(ctypes.byref(h))

    th = threading.Thread(target=probe)  # a fresh thread: nothing has selected a device on it
    th.start()
    th.join()
    assert seen["get"] == 0 and seen["dev"] == InfiniDeviceEnum.CPU
    assert seen["create"] == 5  # INFINI_STATUS_DEVICE_TYPE_NOT_SUPPORTED: there is no CPU backend


def test_null_pointers_are_reported():
    from infinicore_b200.libinfiniop import LIBINFINIOP

    assert LIBINFINIOP.infiniopCreateHandle(None) == 4
    assert LIBINFINIOP.infinirtGetDevice(None, None) == 4
    assert LIBINFINIOP.infiniopGetPagedAttentionWorkspaceSize(None, None) == 4
    assert LIBINFINIOP.infiniopDestroyPagedCachingDescriptor(None) == 4
    # the operators beside the path: a missing handle, descriptor or size pointer is reported, not dereferenced
    from infinicore_b200.libinfiniop import infiniopOperatorDescriptor_t

    d = infiniopOperatorDescriptor_t()
    assert LIBINFINIOP.infiniopCreateRoPEDescriptor(None, ctypes.byref(d), None, None, None, None, None, 0) == 4
    assert LIBINFINIOP.infiniopGetRoPEWorkspaceSize(None, None) == 4
    assert LIBINFINIOP.infiniopRoPE(None, None, 0, None, None, None, None, None, None) == 4
    assert LIBINFINIOP.infiniopDestroyRoPEDescriptor(None) == 4
    assert LIBINFINIOP.infiniopCreateKVCachingDescriptor(None, ctypes.byref(d), None, None, None, None, None) == 4
    assert LIBINFINIOP.infiniopGetKVCachingWorkspaceSize(None, None) == 4
    assert LIBINFINIOP.infiniopKVCaching(None, None, 0, None, None, None, None, None, None) == 4
    assert LIBINFINIOP.infiniopDestroyKVCachingDescriptor(None) == 4
    assert LIBINFINIOP.infiniopCreatePagedDecodeStepRoPEDescriptor(None, ctypes.byref(d), *([None] * 12), 1, 1.0) == 4
    assert LIBINFINIOP.infiniopPagedDecodeStepRoPE(None, None, 0, *([None] * 13)) == 4
    assert LIBINFINIOP.infiniopGetPagedDecodeStepWorkspaceSize(None, None) == 4
    # the kernel status word: no handle, or nowhere to put the flags
    assert LIBINFINIOP.infiniopGetKernelStatus(None, None, None) == 4


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_without_a_gpu_the_runtime_says_so():
    from infinicore_b200.libinfiniop import LIBINFINIOP, InfiniDeviceEnum

    assert LIBINFINIOP.infinirtSetDevice(InfiniDeviceEnum.NVIDIA, 0) == 6  # DEVICE_NOT_FOUND
    assert LIBINFINIOP.infinirtSetDevice(InfiniDeviceEnum.ASCEND, 0) == 5
    n = ctypes.c_int(-1)
    assert LIBINFINIOP.infinirtGetDeviceCount(InfiniDeviceEnum.NVIDIA, ctypes.byref(n)) == 0 and n.value == 0


def test_operators_refuse_cpu_tensors():
    import infinicore_b200 as ib

    q = torch.zeros(1, 1, 64, dtype=torch.float16)
    kc = torch.zeros(1, 1, 16, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ib.paged_attention(q, kc, kc, torch.zeros(1, 1, dtype=torch.int64), torch.ones(1, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ib.paged_caching(kc, kc, q, q, torch.zeros(1, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ib.rope(q, torch.zeros(1, dtype=torch.int64), torch.zeros(4, 32, dtype=torch.float16), torch.zeros(4, 32, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ib.kv_caching(kc, kc, kc[:, :, :1], kc[:, :, :1], torch.zeros(1, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ib.paged_decode_step(q, kc, kc, q, q, torch.zeros(1, 1, dtype=torch.int64), torch.ones(1, dtype=torch.int64))


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from infinicore_b200 import libinfiniop as L

    monkeypatch.setenv("INFINI_ROOT", str(tmp_path))
    monkeypatch.setattr(L, "_PKG", tmp_path)
    with pytest.raises(FileNotFoundError, match="no non-CUDA fallback"):
        L.library_paths()


def test_pybind_module_imports_and_describes_views_without_a_device():
    """The Python module over the C++ host layer: importable on a machine without a GPU (it only links the two
    libraries), tensor views carry shape / strides / dtype, and the reference's operator names are there."""
    from infinicore_b200 import _infinicore_b200 as m

    for name in ("paged_attention", "paged_attention_", "paged_caching_", "Tensor", "DataType", "kernel_status"):
        assert hasattr(m, name)
    t = m.Tensor.from_blob(4096, [2, 3, 4], None, m.DataType.BF16)
    assert t.shape == [2, 3, 4] and t.strides == [12, 4, 1] and t.numel() == 24 and t.data_ptr() == 4096
    s = m.Tensor.from_blob(4096, [3, 2], [1, 3], m.DataType.I64, 1)
    assert s.strides == [1, 3] and s.device_index == 1
    with pytest.raises(ValueError):
        m.Tensor.from_blob(0, [2, 2], [1], m.DataType.F16)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            m.kernel_status()
