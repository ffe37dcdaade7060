"""The C++ host layer (include/infinicore_b200/ops.hpp): descriptor cache, per-stream workspace and exceptions
over the C ABI, as the reference's infinicore operator layer provides them (src/infinicore/ops/infiniop_impl.hpp).

CPU: the header and its test program compile with g++ -Wall -Wextra and link against the built libraries.
GPU: tests/cpp/infinicore_ops_test.cpp runs every wrapper on seeded inputs written here; its outputs are
checked against the CPU oracle (caches bit-exact, attention within fp16 2e-3 / 2e-3, bf16 1e-2 / 1e-2), its
report against the expected cache behaviour (second calls are hits, capture creates nothing, eviction keeps
the cache bounded, a rejected call throws with its status, two more host threads with their own state agree
bit for bit with the main thread)."""
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import ATTN_TOL, assert_close, torch_to_bits
from infinicore_b200 import workloads

ROOT = Path(__file__).resolve().parent.parent
SOURCE = ROOT / "tests" / "cpp" / "infinicore_ops_test.cpp"
LIBDIR = ROOT / "infinicore_b200" / "lib"
CODE = {torch.float16: 12, torch.bfloat16: 19, torch.float32: 13, torch.int64: 6, torch.int32: 5}


def build_program(out_dir: Path) -> Path:
    from infinicore_b200.build import build

    build()
    exe = out_dir / "infinicore_ops_test"
    cmd = ["g++", "-std=c++17", "-O1", "-pthread", "-Wall", "-Wextra", "-Werror", f"-I{ROOT / 'include'}", str(SOURCE), "-o", str(exe),
           f"-L{LIBDIR}", "-linfiniop", "-linfinirt", f"-Wl,-rpath,{LIBDIR}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    return exe


def test_header_and_program_compile_and_link(tmp_path):
    exe = build_program(tmp_path)
    assert exe.is_file()
    # without a directory argument the program only prints its usage (no device call is made)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 2 and "usage" in res.stderr


def write_inputs(directory: Path, tensors: dict, scalars: dict):
    lines = []
    for name, t in tensors.items():
        t = t.contiguous()
        raw = t.view(torch.int16) if t.dtype in (torch.float16, torch.bfloat16) else t
        (directory / f"{name}.bin").write_bytes(raw.numpy().tobytes())
        lines.append(" ".join([name, str(CODE[t.dtype]), str(t.ndim), *map(str, t.shape)]))
    for name, value in scalars.items():
        lines.append(f"scalar {name} {value!r}")
    (directory / "manifest.txt").write_text("\n".join(lines) + "\n")


def read_output(directory: Path, name: str, like: torch.Tensor) -> torch.Tensor:
    raw = np.frombuffer((directory / f"{name}.out.bin").read_bytes(), dtype=np.uint8).copy()
    return torch.from_numpy(raw).view(like.dtype).reshape(like.shape)


@pytest.mark.gpu
def test_every_wrapper_against_the_oracle(tmp_path):
    exe = build_program(tmp_path)
    c = workloads.build_case("cpp", dtype=torch.bfloat16, seq_lens=[300, 17, 1, 160, 2049], num_heads=32, num_kv_heads=8, head_size=128,
                             block_size=16, seed=81)
    pos = c.seq_lens - 1
    table_len = int(pos.max()) + 1
    freqs = 1.0 / (1e4 ** (torch.arange(0, 128, 2).float() / 128))
    angles = torch.outer(torch.arange(table_len).float(), freqs)
    sin, cos = torch.sin(angles).to(c.dtype), torch.cos(angles).to(c.dtype)
    gen = torch.Generator().manual_seed(82)
    kvc_k_cache, kvc_v_cache = torch.randn((3, 4, 16, 64), generator=gen).half(), torch.randn((3, 4, 16, 64), generator=gen).half()
    kvc_k, kvc_v = torch.randn((3, 4, 5, 64), generator=gen).half(), torch.randn((3, 4, 5, 64), generator=gen).half()
    kvc_past = torch.tensor([0, 11, 4], dtype=torch.int64)
    pf = workloads.build_prefill_case("cpp_pf", dtype=torch.float16, new_lens=[70, 5, 130], cached_lens=[0, 33, 64], num_heads=8,
                                      num_kv_heads=2, head_size=128, block_size=16, seed=83)
    write_inputs(tmp_path, {
        "q": c.q, "k_cache": c.k_cache, "v_cache": c.v_cache, "new_k": c.new_k, "new_v": c.new_v, "slot_mapping": c.slot_mapping,
        "block_tables": c.block_tables, "seq_lens": c.seq_lens, "pos_ids": pos, "sin_table": sin, "cos_table": cos,
        "kvc_k_cache": kvc_k_cache, "kvc_v_cache": kvc_v_cache, "kvc_k": kvc_k, "kvc_v": kvc_v, "kvc_past": kvc_past,
        "pf_q": pf.q, "pf_k_cache": pf.k_cache, "pf_v_cache": pf.v_cache, "pf_block_tables": pf.block_tables, "pf_seq_lens": pf.seq_lens,
        "pf_cum": pf.cum_seq_lens_q,
    }, {"scale": float(c.scale), "pf_scale": float(pf.scale)})
    res = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    report = dict(line.split() for line in (tmp_path / "report.txt").read_text().splitlines())
    assert report["ok"] == "1"

    atol, rtol = ATTN_TOL[c.dtype]
    out_like = torch.zeros((c.q.shape[0], c.num_heads, c.v_cache.shape[3]), dtype=c.dtype)
    # A / B / G: caching + attention, one-call step, graph replay
    kb, vb = torch_to_bits(c.k_cache).copy(), torch_to_bits(c.v_cache).copy()
    oracle.paged_caching(kb, vb, torch_to_bits(c.new_k), torch_to_bits(c.new_v), c.slot_mapping.numpy())
    want = oracle.paged_attention(torch_to_bits(c.q), kb, vb, c.block_tables.numpy(), c.seq_lens.numpy(), c.scale, 19)
    for tag in ("a", "b"):
        assert np.array_equal(torch_to_bits(read_output(tmp_path, f"k_cache_{tag}", c.k_cache)), kb), tag
        assert np.array_equal(torch_to_bits(read_output(tmp_path, f"v_cache_{tag}", c.v_cache)), vb), tag
    for tag in ("a", "b", "g", "j0", "j1"):
        assert_close(read_output(tmp_path, f"out_{tag}", out_like).float().numpy(), want, atol, rtol, f"scenario {tag}")
    # C / D: with the rotary embedding
    q_rot = oracle.rope(torch_to_bits(c.q), pos.numpy(), torch_to_bits(sin), torch_to_bits(cos), 19, False)
    k_rot = oracle.rope(torch_to_bits(c.new_k), pos.numpy(), torch_to_bits(sin), torch_to_bits(cos), 19, False)
    kb, vb = torch_to_bits(c.k_cache).copy(), torch_to_bits(c.v_cache).copy()
    oracle.paged_caching(kb, vb, k_rot, torch_to_bits(c.new_v), c.slot_mapping.numpy())
    assert np.array_equal(torch_to_bits(read_output(tmp_path, "q_rot", c.q)), q_rot)
    assert np.array_equal(torch_to_bits(read_output(tmp_path, "k_cache_c", c.k_cache)), kb)
    want = oracle.paged_attention(q_rot, kb, vb, c.block_tables.numpy(), c.seq_lens.numpy(), c.scale, 19)
    assert_close(read_output(tmp_path, "out_c", out_like).float().numpy(), want, atol, rtol, "scenario c")
    # E: contiguous cache append
    want_k, want_v = kvc_k_cache.clone(), kvc_v_cache.clone()
    oracle.kv_caching(want_k.numpy(), want_v.numpy(), kvc_k.numpy(), kvc_v.numpy(), kvc_past.numpy())
    assert torch.equal(read_output(tmp_path, "kvc_k_cache_e", kvc_k_cache), want_k)
    assert torch.equal(read_output(tmp_path, "kvc_v_cache_e", kvc_v_cache), want_v)
    # F: prefill
    want = oracle.paged_attention_prefill(torch_to_bits(pf.q), torch_to_bits(pf.k_cache), torch_to_bits(pf.v_cache), pf.block_tables.numpy(),
                                          pf.seq_lens.numpy(), pf.cum_seq_lens_q.numpy(), pf.scale, 12)
    pf_like = torch.zeros((pf.q.shape[0], pf.num_heads, pf.v_cache.shape[3]), dtype=pf.dtype)
    a16, r16 = ATTN_TOL[pf.dtype]
    assert_close(read_output(tmp_path, "out_pf", pf_like).float().numpy(), want, a16, r16, "prefill")

    # cache behaviour
    assert report["two_call_misses"] == "2" and report["two_call_hits"] == "2"
    assert report["capture_misses"] == "0"
    assert report["workspace_moved"] == "1"  # the stream's workspace grew after the capture; the replays above still ran on theirs
    assert report["kernel_status"] == "0"
    assert int(report["evictions"]) >= 10 and int(report["cached"]) <= int(report["capacity"])
    assert report["error_status"] == "10"
    assert report["cached_after_clear"] == "0"
    assert report["threads"] == "2"
    # the two extra host threads ran the same kernels on the same inputs as scenario A: identical bits
    for tag in ("j0", "j1"):
        assert torch.equal(read_output(tmp_path, f"out_{tag}", out_like).view(torch.int16), read_output(tmp_path, "out_a", out_like).view(torch.int16))
