"""TEST INFRASTRUCTURE.  Compiles the REFERENCE's own sources for the paged decode path into
oracle/_ref/ (libinfinirt.so + libinfiniop.so), for sm_100a, straight from where they lie in the
reference checkout.  Nothing is copied into this repository and the reference's build system
(xmake) is not used: this is a plain nvcc recipe over the ~18 translation units the path needs.

The result is a GPU-side checker and a "reference kernels on the same B200" comparison point:
only tests/ and bench.py's comparison leg load it, through the same C ABI as the product.  The
reference's own ctypes test scripts for these operators are staged beside the libraries
(oracle/_ref/test_infiniop/, verbatim, not committed) so that they can be run against this library.

    python -m oracle.build_ref [/path/to/InfiniCore]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"           # doubles as an $INFINI_ROOT: the libraries land in _ref/lib
LIBDIR = OUT / "lib"
OBJ = OUT / "obj"

RT_SOURCES = ["src/infinirt/infinirt.cc", "src/infinirt/cuda/infinirt_cuda.cu"]
OP_SOURCES = [
    "src/infiniop/tensor_descriptor.cc",
    "src/infiniop/operator_descriptor.cc",
    "src/infiniop/devices/handle.cc",
    "src/infiniop/devices/nvidia/nvidia_common.cu",
    "src/infiniop/ops/paged_attention/operator.cc",
    "src/infiniop/ops/paged_attention/nvidia/paged_attention_nvidia.cu",
    "src/infiniop/ops/paged_attention/nvidia/paged_attention_hd64.cu",
    "src/infiniop/ops/paged_attention/nvidia/paged_attention_hd128.cu",
    "src/infiniop/ops/paged_attention/nvidia/paged_attention_hd192.cu",
    "src/infiniop/ops/paged_attention/nvidia/paged_attention_hd256.cu",
    "src/infiniop/ops/paged_attention/nvidia/paged_attention_hd576.cu",
    "src/infiniop/ops/paged_attention/nvidia/paged_attention_mla_hd576_v512.cu",
    "src/infiniop/ops/paged_attention_prefill/operator.cc",
    "src/infiniop/ops/paged_attention_prefill/nvidia/paged_attention_prefill_nvidia.cu",
    "src/infiniop/ops/paged_caching/operator.cc",
    "src/infiniop/ops/paged_caching/nvidia/paged_caching_nvidia.cu",
    "src/infiniop/ops/kv_caching/operator.cc",
    "src/infiniop/ops/kv_caching/nvidia/kv_caching_nvidia.cu",
    "src/infiniop/ops/rope/operator.cc",
    "src/infiniop/ops/rope/nvidia/rope_nvidia.cu",
    "src/utils/custom_types.cc",
    "src/utils/rearrange.cc",
]
FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-DENABLE_NVIDIA_API",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-w", "-w",
]


def reference_root(arg: str | None = None) -> Path | None:
    # the argument, the environment, or a checkout named `reference` beside this repository
    for cand in (arg, os.getenv("INFINICORE_REFERENCE"), str(Path(__file__).resolve().parent.parent.parent / "reference")):
        if cand and (Path(cand) / "src" / "infiniop" / "ops" / "paged_attention").is_dir():
            return Path(cand)
    return None


def libraries() -> tuple[Path, Path] | None:
    rt, op = LIBDIR / "libinfinirt.so", LIBDIR / "libinfiniop.so"
    return (rt, op) if rt.is_file() and op.is_file() else None


def build(ref: Path | None = None, force: bool = False) -> tuple[Path, Path]:
    ref = ref or reference_root()
    if ref is None:
        raise FileNotFoundError("reference checkout not found")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    OBJ.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{ref / 'include'}", f"-I{ref / 'src'}"]

    def compile_one(rel: str) -> Path:
        src = ref / rel
        obj = OBJ / (rel.replace("/", "_") + ".o")
        stamp = obj.with_suffix(".sha")
        want = hashlib.sha256(src.read_bytes() + " ".join(FLAGS).encode()).hexdigest()
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == want:
            return obj
        cmd = [nvcc, *FLAGS, *inc, "-x", "cu", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"reference source failed to compile: {rel}")
        stamp.write_text(want)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        rt_objs = list(pool.map(compile_one, RT_SOURCES))
        op_objs = list(pool.map(compile_one, OP_SOURCES))
    rt, op = LIBDIR / "libinfinirt.so", LIBDIR / "libinfiniop.so"

    def link(objs, out, extra):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(out), *map(str, objs), "-cudart", "shared", *extra]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"link failed: {out.name}")

    link(rt_objs, rt, [])
    link(op_objs, op, [f"-L{LIBDIR}", "-linfinirt", "-lcublas", "-Xlinker", "-rpath=$ORIGIN"])
    stage_test_harness(ref)
    return rt, op


# The reference's own ctypes test harness for this path (test/infiniop/libinfiniop + the operators' test
# scripts), staged verbatim next to the libraries built from its sources - like them an artefact of the
# reference checkout that lives only under oracle/_ref/ and is never committed.  tests/ref_harness.py runs
# these scripts against THIS library (the drop-in claim: the reference's tests, unmodified, pass on it).
HARNESS = OUT / "test_infiniop"
HARNESS_SCRIPTS = ["paged_attention.py", "paged_caching.py", "paged_attention_prefill.py", "rope.py", "kv_caching.py"]


def stage_test_harness(ref: Path) -> Path | None:
    src = ref / "test" / "infiniop"
    if not (src / "libinfiniop").is_dir():
        return None
    (HARNESS / "libinfiniop").mkdir(parents=True, exist_ok=True)
    for f in (src / "libinfiniop").glob("*.py"):
        shutil.copyfile(f, HARNESS / "libinfiniop" / f.name)
    for name in HARNESS_SCRIPTS:
        if (src / name).is_file():
            shutil.copyfile(src / name, HARNESS / name)
    return HARNESS


if __name__ == "__main__":
    root = reference_root(sys.argv[1] if len(sys.argv) > 1 else None)
    print(build(root, force="--force" in sys.argv))
