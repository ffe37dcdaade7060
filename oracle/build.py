"""TEST INFRASTRUCTURE.  Builds the CPU oracle (oracle/paged_oracle.c, oracle/rope_oracle.c) into
oracle/_build/libpaged_oracle.so with gcc + OpenMP.

    python -m oracle.build
"""
from __future__ import annotations

import hashlib
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCES = [HERE / "paged_oracle.c", HERE / "rope_oracle.c"]
OUT_DIR = HERE / "_build"
OUT = OUT_DIR / "libpaged_oracle.so"
FLAGS = ["-O3", "-march=x86-64-v2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-Wall", "-Wextra"]


def build(force: bool = False) -> Path:
    OUT_DIR.mkdir(exist_ok=True)
    stamp = OUT_DIR / "libpaged_oracle.sha"
    want = hashlib.sha256(b"".join(src.read_bytes() for src in SOURCES) + " ".join(FLAGS).encode()).hexdigest()
    if not force and OUT.exists() and stamp.exists() and stamp.read_text() == want:
        return OUT
    cmd = ["gcc", *FLAGS, *map(str, SOURCES), "-o", str(OUT), "-lm"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("gcc failed on the oracle")
    stamp.write_text(want)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
