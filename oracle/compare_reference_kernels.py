"""Times this library's paged attention against the reference's own kernels (oracle/_ref, built
by oracle/build_ref.py) on the benchmark configurations and a few other shapes, each library in a
child process of its own (they export the same symbols).  Prints one JSON line per (configuration,
library, environment).  This is what the tables under profiles/ that compare the two were made with;
it is a checker's tool like the rest of this folder - nothing in the library uses it.

    python oracle/compare_reference_kernels.py [c1 c2 c3 c4 b1 b8 b1long g16 h64 h192 h256 h576 mla mla37 p1 p2]
"""
import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
REF_ROOT = ROOT / "oracle" / "_ref"

SPECS = {
    "c1": {"builder": "config1_small", "kwargs": {}},
    "c2": {"builder": "config2_llama8b", "kwargs": {"device": "cuda"}},
    "c3": {"builder": "config3_ragged72b", "kwargs": {"device": "cuda"}},
    "c4": {"builder": "config4_longctx", "kwargs": {"device": "cuda"}},
    # small batches, Llama-3-8B heads: one sequence of 4096 tokens; eight of 1024; one of 65536
    "b1": {"builder": "build_case", "kwargs": {"name": "b1", "dtype": "bfloat16", "seq_lens": [4096], "num_heads": 32, "num_kv_heads": 8,
                                               "head_size": 128, "block_size": 16, "seed": 11, "device": "cuda"}},
    "b8": {"builder": "build_case", "kwargs": {"name": "b8", "dtype": "bfloat16", "seq_lens": [1024] * 8, "num_heads": 32, "num_kv_heads": 8,
                                               "head_size": 128, "block_size": 16, "seed": 12, "device": "cuda"}},
    "b1long": {"builder": "build_case", "kwargs": {"name": "b1long", "dtype": "bfloat16", "seq_lens": [65536], "num_heads": 32, "num_kv_heads": 8,
                                                   "head_size": 128, "block_size": 16, "seed": 13, "device": "cuda"}},
    # 16 q-heads per kv-head (Llama-3.1-405B grouping): 128 / 8 heads, 64 sequences x 4096 tokens
    "g16": {"builder": "build_case", "kwargs": {"name": "g16", "dtype": "bfloat16", "seq_lens": [4096] * 64, "num_heads": 128, "num_kv_heads": 8,
                                                "head_size": 128, "block_size": 16, "seed": 16, "device": "cuda"}},
    # the other head sizes the descriptor accepts: 64 sequences x 4096 tokens each
    "h64": {"builder": "build_case", "kwargs": {"name": "h64", "dtype": "float16", "seq_lens": [4096] * 64, "num_heads": 32, "num_kv_heads": 8,
                                                "head_size": 64, "block_size": 16, "seed": 64, "device": "cuda"}},
    "h192": {"builder": "build_case", "kwargs": {"name": "h192", "dtype": "bfloat16", "seq_lens": [4096] * 64, "num_heads": 32, "num_kv_heads": 8,
                                                 "head_size": 192, "block_size": 16, "seed": 192, "device": "cuda"}},
    "h256": {"builder": "build_case", "kwargs": {"name": "h256", "dtype": "bfloat16", "seq_lens": [4096] * 64, "num_heads": 16, "num_kv_heads": 8,
                                                 "head_size": 256, "block_size": 16, "seed": 256, "device": "cuda"}},
    "h576": {"builder": "build_case", "kwargs": {"name": "h576", "dtype": "bfloat16", "seq_lens": [4096] * 64, "num_heads": 16, "num_kv_heads": 1,
                                                 "head_size": 576, "block_size": 16, "seed": 576, "std": 0.3, "device": "cuda"}},
    # latent attention: keys 576 wide, values 512 wide, one shared kv-head, 128 query heads
    "mla": {"builder": "build_case", "kwargs": {"name": "mla", "dtype": "bfloat16", "seq_lens": [4096] * 64, "num_heads": 128, "num_kv_heads": 1,
                                                "head_size": 576, "value_size": 512, "block_size": 16, "seed": 577, "std": 0.3, "device": "cuda"}},
    # the same with 37 sequences: 37 x 8 head tiles = 296 units, one per worker of the wide kernel, so the eight head
    # tiles of a sequence walk the same tokens at the same time (what the L2 does for them shows in an ncu capture)
    "mla37": {"builder": "build_case", "kwargs": {"name": "mla37", "dtype": "bfloat16", "seq_lens": [4096] * 37, "num_heads": 128, "num_kv_heads": 1,
                                                  "head_size": 576, "value_size": 512, "block_size": 16, "seed": 578, "std": 0.3, "device": "cuda"}},
    # prefill, Llama-3-8B head shape: 8 prompts x 2048 new tokens; and 4 x 1024 new over 3072 cached
    "p1": {"builder": "prefill_llama8b", "kwargs": {"device": "cuda", "num_seqs": 8, "new_len": 2048, "cached_len": 0}},
    "p2": {"builder": "prefill_llama8b", "kwargs": {"device": "cuda", "num_seqs": 4, "new_len": 1024, "cached_len": 3072}},
}


def run(spec, env_extra, reference):
    env = dict(os.environ)
    env.pop("INFINI_ROOT", None)
    if reference:
        env["INFINI_ROOT"] = str(REF_ROOT)
    env.update(env_extra)
    with tempfile.TemporaryDirectory() as tmp:
        out = Path(tmp) / "o.pt"
        res = subprocess.run([sys.executable, str(ROOT / "tests" / "ref_runner.py"), json.dumps(spec), str(out)],
                             env=env, capture_output=True, text=True, timeout=900)
        if res.returncode != 0:
            return {"error": (res.stdout + res.stderr)[-500:]}
        return torch.load(out)


def main():
    names = sys.argv[1:] or ["c2", "c3", "c4"]
    for name in names:
        spec = dict(SPECS[name], iters=30, caching=False)
        if name.startswith("p"):
            runs = [("this library (default path)", False, {}),
                    ("this library, tcgen05 kernel", False, {"INFINIOP_PAGED_PREFILL_PATH": "umma"}),
                    ("this library, mma.sync tile kernel", False, {"INFINIOP_PAGED_PREFILL_PATH": "tiles"}),
                    ("this library, row-wise generic kernel", False, {"INFINIOP_PAGED_PREFILL_PATH": "generic"}),
                    ("reference kernels, default", True, {})]
        else:
            runs = [("this library", False, {}),
                    ("reference kernels, default (split-KV CTA, 4 splits)", True, {}),
                    ("reference kernels, INFINIOP_FLASH_DECODE_SPLITKV=0", True, {"INFINIOP_FLASH_DECODE_SPLITKV": "0"})]
        base = None
        for label, reference, env in runs:
            r = run(spec, env, reference)
            line = {"config": name, "library": label}
            if "error" in r:
                line["error"] = r["error"]
            else:
                line.update(attn_ms=r["attn_ms"], workspace_bytes=r["workspace"])
                if "kv_bytes" in r:
                    line["kv_GBps"] = r["kv_bytes"] / r["attn_ms"] / 1e6
                if "flops" in r:
                    line["TFLOPs"] = r["flops"] / r["attn_ms"] / 1e9
                if base is None:
                    base = r["out"].float()
                else:
                    line["max_abs_diff_vs_this_library"] = float((r["out"].float() - base).abs().max())
            print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
