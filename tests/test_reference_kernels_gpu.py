"""GPU parity against the REFERENCE'S OWN KERNELS: the reference's CUDA sources for this path,
compiled for sm_100a into oracle/_ref by oracle/build_ref.py, run in a child process on the same
seeded inputs as this library.  paged_caching must agree bit for bit; attention within the path's
tolerance (fp16 2e-3 / 2e-3, bf16 1e-2 / 1e-2).  Skipped when oracle/_ref was not built."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import ATTN_TOL, assert_close

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF_ROOT = ROOT / "oracle" / "_ref"


def run(spec, tmp_path, reference: bool):
    env = dict(os.environ)
    env.pop("INFINI_ROOT", None)
    if reference:
        env["INFINI_ROOT"] = str(REF_ROOT)
    out = tmp_path / ("ref.pt" if reference else "mine.pt")
    res = subprocess.run([sys.executable, str(ROOT / "tests" / "ref_runner.py"), json.dumps(spec), str(out)],
                         env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return torch.load(out)


SPECS = [
    {"builder": "config1_small", "kwargs": {"seed": 1, "device": "cpu"}},
    {"builder": "build_case", "kwargs": {"name": "gqa4", "dtype": "bfloat16", "seq_lens": [300, 17, 1, 160, 1000], "num_heads": 32,
                                          "num_kv_heads": 8, "head_size": 128, "block_size": 16, "seed": 51}},
    {"builder": "build_case", "kwargs": {"name": "gqa8", "dtype": "float16", "seq_lens": [64, 333, 16, 15, 2047], "num_heads": 64,
                                          "num_kv_heads": 8, "head_size": 128, "block_size": 16, "seed": 52, "std": 0.5}},
    {"builder": "build_case", "kwargs": {"name": "mha64", "dtype": "float16", "seq_lens": [77, 500], "num_heads": 8,
                                          "num_kv_heads": 8, "head_size": 64, "block_size": 16, "seed": 53}},
    {"builder": "config2_llama8b", "kwargs": {"seed": 2, "device": "cuda", "num_seqs": 16}},
]


@pytest.mark.skipif(not (REF_ROOT / "lib" / "libinfiniop.so").is_file(), reason="oracle/_ref not built")
@pytest.mark.parametrize("spec", SPECS, ids=lambda s: s["kwargs"].get("name", s["builder"]))
def test_same_inputs_same_results_as_the_reference_kernels(spec, tmp_path):
    spec = dict(spec, return_cache=spec["builder"] != "config2_llama8b")
    ref = run(spec, tmp_path, reference=True)
    mine = run(spec, tmp_path, reference=False)
    assert "oracle/_ref" in ref["library"] and "oracle/_ref" not in mine["library"]
    if spec["return_cache"]:
        assert torch.equal(ref["k_cache"].view(torch.int16), mine["k_cache"].view(torch.int16)), "paged_caching differs"
        assert torch.equal(ref["v_cache"].view(torch.int16), mine["v_cache"].view(torch.int16)), "paged_caching differs"
    atol, rtol = ATTN_TOL[ref["out"].dtype]
    assert_close(mine["out"].float().numpy(), ref["out"].float().numpy(), atol, rtol, "vs reference kernels")


PREFILL_SPECS = [
    {"builder": "build_prefill_case", "kwargs": {"name": "pf_mha", "dtype": "bfloat16", "new_lens": [70, 5, 130], "cached_lens": [0, 33, 64],
                                                  "num_heads": 8, "num_kv_heads": 8, "head_size": 128, "block_size": 16, "seed": 54}},
    {"builder": "build_prefill_case", "kwargs": {"name": "pf_gqa4", "dtype": "float16", "new_lens": [200, 64, 1], "cached_lens": [17, 0, 300],
                                                  "num_heads": 32, "num_kv_heads": 8, "head_size": 128, "block_size": 16, "seed": 55}},
    {"builder": "build_prefill_case", "kwargs": {"name": "pf_bs8", "dtype": "bfloat16", "new_lens": [16, 9, 64], "cached_lens": [0, 7, 30],
                                                  "num_heads": 4, "num_kv_heads": 4, "head_size": 128, "block_size": 8, "seed": 56}},
]


@pytest.mark.skipif(not (REF_ROOT / "lib" / "libinfiniop.so").is_file(), reason="oracle/_ref not built")
@pytest.mark.parametrize("spec", PREFILL_SPECS, ids=lambda s: s["kwargs"]["name"])
def test_prefill_same_results_as_the_reference_kernels(spec, tmp_path):
    ref = run(spec, tmp_path, reference=True)
    mine = run(spec, tmp_path, reference=False)
    assert "oracle/_ref" in ref["library"] and "oracle/_ref" not in mine["library"]
    atol, rtol = ATTN_TOL[ref["out"].dtype]
    assert_close(mine["out"].float().numpy(), ref["out"].float().numpy(), atol, rtol, "prefill vs reference kernels")


# the reference test's tolerances for this operator (test/infiniop/rope.py:46-50); its CUDA kernel computes
# in the tensor's own 16-bit type, this library in fp32 with one rounding
ROPE_TOL = {torch.float16: (1e-3, 1e-2), torch.bfloat16: (5e-3, 5e-2), torch.float32: (1e-4, 1e-3)}
ROPE_SPECS = [
    {"op": "rope", "shape": [10, 32, 64], "dtype": "float16", "algo": 0, "seed": 61, "table_len": 64},
    {"op": "rope", "shape": [11, 33, 128], "dtype": "bfloat16", "algo": 1, "seed": 62, "table_len": 64},
    {"op": "rope", "shape": [8, 10, 32, 64], "dtype": "float32", "algo": 1, "seed": 63, "table_len": 32},
    {"op": "rope", "shape": [8192, 32, 128], "dtype": "bfloat16", "algo": 1, "seed": 64, "table_len": 8192, "iters": 20},
]


@pytest.mark.skipif(not (REF_ROOT / "lib" / "libinfiniop.so").is_file(), reason="oracle/_ref not built")
@pytest.mark.parametrize("spec", ROPE_SPECS, ids=lambda s: "x".join(map(str, s["shape"])) + s["dtype"])
def test_rope_same_results_as_the_reference_kernel(spec, tmp_path):
    ref = run(spec, tmp_path, reference=True)
    mine = run(spec, tmp_path, reference=False)
    assert "oracle/_ref" in ref["library"] and "oracle/_ref" not in mine["library"]
    atol, rtol = ROPE_TOL[ref["y"].dtype]
    a, b = mine["y"].float().numpy(), ref["y"].float().numpy()
    if a.size < 1 << 20:
        assert_close(a, b, atol, rtol, "rope vs reference kernel")
    else:
        # Among millions of pairs a few have products that cancel (x0 cos ~ x1 sin): the reference kernel rounds
        # each product to the 16-bit type first, so its difference carries up to 2^-8 of the products (|x| up to ~5)
        # there, while this library's fp32 arithmetic (bit-exact against the oracle in test_rope_gpu.py) does not.
        err = np.abs(a - b)
        outside = err > atol + rtol * np.abs(b)
        assert outside.mean() < 1e-5 and err.max() < 0.05, (int(outside.sum()), float(err.max()))
    if "ms" in ref:
        print(f"rope {spec['shape']}: reference {ref['ms'] * 1e3:.1f} us, this library {mine['ms'] * 1e3:.1f} us "
              f"({mine['bytes'] / mine['ms'] / 1e6:.0f} GB/s)")


KV_CACHING_SPECS = [
    {"op": "kv_caching", "shape": [8, 8, 64, 32], "seq_len": 5, "dtype": "bfloat16", "seed": 71},
    {"op": "kv_caching", "shape": [2, 4, 32, 16], "seq_len": 31, "dtype": "float32", "seed": 72},
    # a prefill-sized append: 16 sequences x 8 heads x 2048 new rows of 128 (134 MB of rows in and out)
    {"op": "kv_caching", "shape": [16, 8, 2048, 128], "seq_len": 2048, "dtype": "bfloat16", "seed": 73, "iters": 20},
]


@pytest.mark.skipif(not (REF_ROOT / "lib" / "libinfiniop.so").is_file(), reason="oracle/_ref not built")
@pytest.mark.parametrize("spec", KV_CACHING_SPECS, ids=lambda s: "x".join(map(str, s["shape"])) + s["dtype"])
def test_kv_caching_same_results_as_the_reference_kernel(spec, tmp_path):
    ref = run(spec, tmp_path, reference=True)
    mine = run(spec, tmp_path, reference=False)
    assert "oracle/_ref" in ref["library"] and "oracle/_ref" not in mine["library"]
    for name in ("k_cache", "v_cache"):
        a, b = mine[name], ref[name]
        view = torch.int16 if a.element_size() == 2 else torch.int32
        assert torch.equal(a.view(view), b.view(view)), f"{name} differs from the reference kernel's"
    if "ms" in ref:
        print(f"kv_caching {spec['shape']}: reference {ref['ms'] * 1e3:.1f} us, this library {mine['ms'] * 1e3:.1f} us "
              f"({mine['bytes'] / mine['ms'] / 1e6:.0f} GB/s)")


PAGED_CACHING_SPECS = [
    # a prefill-sized scatter: 8 prompts x 2048 tokens, 8 kv-heads, head 128 (134 MB of rows in, 134 MB out)
    {"op": "paged_caching", "tokens": 16384, "kv_heads": 8, "head": 128, "block": 16, "dtype": "bfloat16", "seed": 74, "iters": 20},
    {"op": "paged_caching", "tokens": 1000, "kv_heads": 2, "head": 64, "block": 32, "dtype": "float16", "seed": 75},
]


@pytest.mark.skipif(not (REF_ROOT / "lib" / "libinfiniop.so").is_file(), reason="oracle/_ref not built")
@pytest.mark.parametrize("spec", PAGED_CACHING_SPECS, ids=lambda s: f"{s['tokens']}x{s['kv_heads']}x{s['head']}")
def test_prefill_sized_paged_caching_same_as_the_reference_kernel(spec, tmp_path):
    ref = run(spec, tmp_path, reference=True)
    mine = run(spec, tmp_path, reference=False)
    assert "oracle/_ref" in ref["library"] and "oracle/_ref" not in mine["library"]
    for name in ("k_cache", "v_cache"):
        assert torch.equal(mine[name].view(torch.int16), ref[name].view(torch.int16)), f"{name} differs from the reference kernel's"
    if "ms" in ref:
        print(f"paged_caching {spec['tokens']} tokens: reference {ref['ms'] * 1e3:.1f} us, this library {mine['ms'] * 1e3:.1f} us "
              f"({mine['bytes'] / mine['ms'] / 1e6:.0f} GB/s)")
