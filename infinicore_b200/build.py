"""Builds libinfinirt.so and libinfiniop.so for sm_100a with nvcc, in-tree.

The reference builds the same two libraries with xmake (xmake.lua, xmake/nvidia.lua);
xmake is not a dependency here - this script is the build.  Output goes to
infinicore_b200/lib/, which doubles as $INFINI_ROOT/lib for loaders that follow the
reference's layout (test/infiniop/libinfiniop/liboperators.py:11-56).

    python -m infinicore_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
LIB = PKG / "lib"
OBJ = PKG / "build"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = [
    "-std=c++17",
    "-O3",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC,-fvisibility=hidden,-Wall",
    "--expt-relaxed-constexpr",
    f"-I{INCLUDE}",
    f"-I{CSRC}",
]

RT_SOURCES = ["runtime/infinirt.cu"]
OP_SOURCES = [
    "handle.cu",
    "kernel_status.cu",
    "paged_caching/paged_caching.cu",
    "paged_attention/operator.cu",
    "paged_attention/decode_generic.cu",
    "paged_attention/decode_stream.cu",
    "paged_attention/static_workspace.cu",
    "paged_attention/decode_step.cu",
    "rope/rope.cu",
    "kv_caching/kv_caching.cu",
    "paged_attention_prefill/operator.cu",
    "paged_attention_prefill/prefill_generic.cu",
    "paged_attention_prefill/prefill_tiles.cu",
    "paged_attention_prefill/prefill_umma.cu",
]


# libinfiniccl: the InfiniCCL C ABI over NCCL (system libnccl: /usr/include/nccl.h, -lnccl)
CCL_SOURCES = ["ccl/infiniccl.cu"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; this library has no non-CUDA build")
    return exe


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(p.read_bytes())
    h.update(" ".join(COMMON + ARCH_FLAGS).encode())
    return h.hexdigest()


def _headers():
    return list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(INCLUDE.rglob("*.h"))


def _compile(src: str, verbose: bool, extra=()) -> Path:
    src_path = CSRC / src
    obj = OBJ / (src.replace("/", "_") + ".o")
    stamp = obj.with_suffix(".sha")
    want = _digest([src_path] + _headers())
    if obj.exists() and stamp.exists() and stamp.read_text() == want:
        return obj
    cmd = [nvcc(), *COMMON, *ARCH_FLAGS, *extra, "-c", str(src_path), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}")
    stamp.write_text(want)
    return obj


def _link(objs, out: Path, extra, verbose: bool) -> None:
    cmd = [nvcc(), "-shared", *ARCH_FLAGS, "-o", str(out), *map(str, objs), "-cudart", "shared", *extra]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"link failed for {out.name}")


def build(force: bool = False, verbose: bool = False) -> dict:
    """Compiles what is stale and returns {"infinirt": path, "infiniop": path, "infiniccl": path, "pybind": path}."""
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    if force:
        for f in OBJ.glob("*.sha"):
            f.unlink()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        rt_objs = list(pool.map(lambda s: _compile(s, verbose), RT_SOURCES))
        op_objs = list(pool.map(lambda s: _compile(s, verbose), OP_SOURCES))
        ccl_objs = list(pool.map(lambda s: _compile(s, verbose), CCL_SOURCES))
    librt = LIB / "libinfinirt.so"
    libop = LIB / "libinfiniop.so"
    libccl = LIB / "libinfiniccl.so"
    newest_obj = max(o.stat().st_mtime for o in rt_objs + op_objs + ccl_objs)
    if force or not librt.exists() or librt.stat().st_mtime < newest_obj:
        _link(rt_objs, librt, ["-ldl"], verbose)
    if force or not libop.exists() or libop.stat().st_mtime < newest_obj:
        _link(op_objs, libop, [f"-L{LIB}", "-linfinirt", "-Xlinker", "-rpath=$ORIGIN"], verbose)
    if force or not libccl.exists() or libccl.stat().st_mtime < newest_obj:
        _link(ccl_objs, libccl, [f"-L{LIB}", "-linfinirt", "-lnccl", "-Xlinker", "-rpath=$ORIGIN"], verbose)
    return {"infinirt": librt, "infiniop": libop, "infiniccl": libccl, "pybind": build_pybind(force, verbose)}


def build_pybind(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the Python module over the C++ host layer (csrc/pybind/module.cpp) with g++ and pybind11,
    in-tree, linked to the libraries in lib/ (found again at run time through $ORIGIN/lib)."""
    import sysconfig

    import pybind11

    src = CSRC / "pybind" / "module.cpp"
    out = PKG / ("_infinicore_b200" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
    stamp = OBJ / "pybind_module.sha"
    want = _digest([src, INCLUDE / "infinicore_b200" / "ops.hpp"] + list(INCLUDE.rglob("*.h")))
    newest_lib = max((LIB / n).stat().st_mtime for n in ("libinfinirt.so", "libinfiniop.so"))
    if not force and out.exists() and stamp.exists() and stamp.read_text() == want and out.stat().st_mtime >= newest_lib:
        return out
    gxx = shutil.which("g++")
    if gxx is None:
        raise RuntimeError("g++ not found")
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra",
           f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{INCLUDE}",
           str(src), "-o", str(out), f"-L{LIB}", "-linfiniop", "-linfinirt", "-Wl,-rpath,$ORIGIN/lib"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("g++ failed on pybind/module.cpp")
    stamp.write_text(want)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="echo commands and ptxas resource usage")
    args = ap.parse_args()
    out = build(force=args.force, verbose=args.verbose)
    for k, v in out.items():
        print(f"{k}: {v}")


if __name__ == "__main__":
    main()
