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
    # no collective has run in these processes: the communication members are valid and say so
    assert s["valid_fields"] & 16 and s["communication_bytes"] == 0 and s["communication_time_ratio"] == 0


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc for the stand-in library")
def test_utilisation_comes_from_the_management_library(tmp_path):
    fake = tmp_path / "libfake_management.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(fake), str(ROOT / "tests" / "cpp" / "fake_management_library.c")], check=True)
    s = snapshot(fake)
    check_memory(s)
    assert s["valid_fields"] == 1 | 2 | 4 | 8 | 16
    assert s["estimated_fields"] == 8  # the kernel-time ratio is the compute sample again
    assert abs(s["compute_utilization"] - 0.37) < 1e-6 and abs(s["memory_bandwidth_utilization"] - 0.12) < 1e-6
    assert abs(s["kernel_time_ratio"] - 0.37) < 1e-6


def test_without_a_management_library_only_memory_is_flagged(tmp_path):
    s = snapshot(tmp_path / "no_such_library.so")
    check_memory(s)
    assert s["valid_fields"] == 1 | 16 and s["estimated_fields"] == 0
    assert s["compute_utilization"] == 0 and s["memory_bandwidth_utilization"] == 0


def test_with_the_machines_own_library():
    s = snapshot()
    check_memory(s)
    if s["valid_fields"] & 2:
        assert s["valid_fields"] & 4 and s["valid_fields"] & 8
        assert 0.0 <= s["compute_utilization"] <= 1.0 and 0.0 <= s["memory_bandwidth_utilization"] <= 1.0


COMM_CHILD = r"""
import ctypes, json, sys, time
sys.path.insert(0, %r)
import torch
from infinicore_b200 import ccl
from infinicore_b200.libinfiniop import LIBINFINIOP

class Snapshot(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int), ("device_id", ctypes.c_int), ("valid_fields", ctypes.c_uint64),
                ("estimated_fields", ctypes.c_uint64), ("free_bytes", ctypes.c_size_t), ("total_bytes", ctypes.c_size_t),
                ("used_bytes", ctypes.c_size_t), ("reserved_bytes", ctypes.c_size_t), ("compute_utilization", ctypes.c_float),
                ("memory_bandwidth_utilization", ctypes.c_float), ("kernel_time_ratio", ctypes.c_float),
                ("communication_time_ratio", ctypes.c_float), ("communication_bytes", ctypes.c_uint64)]

fn = LIBINFINIOP.librt.infinirtGetDeviceResourceSnapshot
fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(Snapshot)]

def snap():
    s = Snapshot()
    assert fn(1, 0, ctypes.byref(s)) == 0
    return {"valid": s.valid_fields, "bytes": s.communication_bytes, "ratio": s.communication_time_ratio}

torch.cuda.set_device(0)
comm = ccl.init_all([0])[0]
n = 16 << 20                                   # 64 MiB of fp32 per collective
x = torch.ones(n, dtype=torch.float32, device="cuda:0")
y = torch.empty_like(x)
out = {"before": snap()}
for _ in range(3):
    comm.all_reduce(x, y)                      # three samples of 64 MiB each
comm.group_start()                             # a caller's group is one sample carrying the sum of its payloads
comm.broadcast(x[: n // 2], y[: n // 2], 0)
comm.broadcast(x[n // 2:], y[n // 2:], 0)
comm.group_end()
torch.cuda.synchronize()
out["after"] = snap()
out["sum_ok"] = bool((y == 1).all())
# captured collectives are not sampled (their events could not be read back)
g = torch.cuda.CUDAGraph()
side = torch.cuda.Stream()
with torch.cuda.stream(side):
    comm.all_reduce(x, y)
    side.synchronize()
    before_capture = snap()["bytes"]
    with torch.cuda.graph(g, stream=side):
        comm.all_reduce(x, y)
    g.replay()
    side.synchronize()
out["captured_added"] = snap()["bytes"] - before_capture
time.sleep(1.3)                                # the window is one second
out["later"] = snap()
torch.cuda.synchronize()
comm.destroy()
print(json.dumps(out))
""" % str(ROOT)


def test_collectives_show_up_in_the_communication_members():
    import os

    env = dict(os.environ)
    env.pop("INFINIRT_MANAGEMENT_LIBRARY", None)
    res = subprocess.run([sys.executable, "-c", COMM_CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    r = json.loads(res.stdout.strip().splitlines()[-1])
    assert r["sum_ok"]
    assert r["before"]["valid"] & 16 and r["before"]["bytes"] == 0
    assert r["after"]["valid"] & 16
    assert r["after"]["bytes"] == 4 * (64 << 20), "three all-reduces of 64 MiB and one group of two 32 MiB broadcasts"
    assert 0.0 < r["after"]["ratio"] <= 1.0
    assert r["captured_added"] == 0
    assert r["later"]["bytes"] == 0 and r["later"]["ratio"] == 0, "samples older than a second leave the window"
