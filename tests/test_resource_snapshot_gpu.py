"""infinirtGetDeviceResourceSnapshot: memory capacity from the CUDA runtime, utilisation from the driver's
management library looked up at run time (reference src/infinirt/cuda/infinirt_cuda.cu:163-352).  The library
is chosen once per process, so every case runs in a child process: with a stand-in library that answers fixed
figures, with a name that does not load, and with whatever the machine really has."""
import json
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

CHILD = r"""
import ctypes, json, sys
sys.path.insert(0, %r)
from infinicore_b200.libinfiniop import LIBINFINIOP

class Snapshot(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int), ("device_id", ctypes.c_int), ("valid_fields", ctypes.c_uint64),
                ("estimated_fields", ctypes.c_uint64), ("free_bytes", ctypes.c_size_t), ("total_bytes", ctypes.c_size_t),
                ("used_bytes", ctypes.c_size_t), ("reserved_bytes", ctypes.c_size_t), ("compute_utilization", ctypes.c_float),
                ("memory_bandwidth_utilization", ctypes.c_float), ("kernel_time_ratio", ctypes.c_float),
                ("communication_time_ratio", ctypes.c_float), ("communication_bytes", ctypes.c_uint64)]

fn = LIBINFINIOP.librt.infinirtGetDeviceResourceSnapshot
fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(Snapshot)]
snap = Snapshot()
status = fn(1, 0, ctypes.byref(snap))
null_status = fn(1, 0, None)
print(json.dumps({"status": status, "null_status": null_status, **{k: getattr(snap, k) for k, _ in Snapshot._fields_}}))
""" % str(ROOT)


def snapshot(env_library=None):
    import os

    env = dict(os.environ)
    env.pop("INFINIRT_MANAGEMENT_LIBRARY", None)
    if env_library is not None:
        env["INFINIRT_MANAGEMENT_LIBRARY"] = str(env_library)
    res = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    return json.loads(res.stdout.strip().splitlines()[-1])


def check_memory(s):
    assert s["status"] == 0 and s["null_status"] == 4  # INFINI_STATUS_NULL_POINTER
    assert s["device_type"] == 1 and s["device_id"] == 0
    assert s["valid_fields"] & 1 and s["total_bytes"] > (100 << 30) and s["used_bytes"] == s["total_bytes"] - s["free_bytes"]
    assert s["valid_fields"] & 16 == 0 and s["communication_bytes"] == 0  # no collective-timing store on this path


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc for the stand-in library")
def test_utilisation_comes_from_the_management_library(tmp_path):
    fake = tmp_path / "libfake_management.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(fake), str(ROOT / "tests" / "cpp" / "fake_management_library.c")], check=True)
    s = snapshot(fake)
    check_memory(s)
    assert s["valid_fields"] == 1 | 2 | 4 | 8
    assert s["estimated_fields"] == 8  # the kernel-time ratio is the compute sample again
    assert abs(s["compute_utilization"] - 0.37) < 1e-6 and abs(s["memory_bandwidth_utilization"] - 0.12) < 1e-6
    assert abs(s["kernel_time_ratio"] - 0.37) < 1e-6


def test_without_a_management_library_only_memory_is_flagged(tmp_path):
    s = snapshot(tmp_path / "no_such_library.so")
    check_memory(s)
    assert s["valid_fields"] == 1 and s["estimated_fields"] == 0
    assert s["compute_utilization"] == 0 and s["memory_bandwidth_utilization"] == 0


def test_with_the_machines_own_library():
    s = snapshot()
    check_memory(s)
    if s["valid_fields"] & 2:
        assert s["valid_fields"] & 4 and s["valid_fields"] & 8
        assert 0.0 <= s["compute_utilization"] <= 1.0 and 0.0 <= s["memory_bandwidth_utilization"] <= 1.0
