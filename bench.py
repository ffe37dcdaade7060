#!/usr/bin/env python
"""Benchmark of the paged decode hot path: one step = infiniopPagedCaching (the newest token's
K/V rows) followed by infiniopPagedAttention over the paged KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--blocks R] [--workload c2|c3|c4|c5] [--impl reference]

One JSON line on stdout (rank 0).  `value` is KV-read bandwidth of the whole job in GB/s:
algorithmic KV bytes of one step (every K and V element of every live token once, independent of
the GQA group size and of how the work is split) summed over all ranks, divided by the device-timed
step (max over ranks).  The timed region is R blocks of K back-to-back steps, each block bracketed by
a barrier and a synchronize; `ms_per_step` is the median block (min and max beside it).  Multi-GPU
runs shard by sequence: every rank owns its sequences, its block tables and its own cache pool; there
is no data-path collective (scaling "weak": each rank runs a full copy of the workload with its own
seed; workload c5 instead splits one 2048-sequence batch round-robin, "strong").

Side records in the same line (each guarded: a failure costs the record, never the headline): the
ragged and the long-context configurations on one GPU (`c3`, `c4`), the 2048-sequence batch split
over the N ranks under two placement policies (`c5_strong`), at N > 1 the KV-head-sharded mode with
its two ways of combining the outputs (`head_sharded`), and at N = 1 the reference's own CUDA kernels
on the same inputs (`reference_gpu`, a child process, only where oracle/_ref was built).

`--impl reference` times the CPU restatement of the reference's checker (oracle/, all host
threads) on the same workload; only rank 0 works.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "paged_attn_decode_kv_read_bandwidth"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, taken from one ncu
# capture of this workload.  A capture describes the kernel source it was taken from: the entry is only
# reported while that source file still has the recorded hash, so it cannot silently go stale.
NCU_TRAFFIC = {
    "c2": {"bytes": 1077984000 + 4757000, "kernel": "pagedDecodeStreamKernel<bf16,128,8,pool off>", "captured": "2026-11-25",
           "source": "infinicore_b200/csrc/paged_attention/decode_stream.cu", "source_sha256_16": "d799af565937714a"},
}


def ncu_traffic(workload):
    """(bytes per launch or None, provenance string)."""
    import hashlib

    rec = NCU_TRAFFIC.get(workload)
    if rec is None:
        return None, "no ncu capture of this workload"
    try:
        now = hashlib.sha256((ROOT / rec["source"]).read_bytes()).hexdigest()[:16]
    except OSError:
        now = None
    if now != rec["source_sha256_16"]:
        return None, f"ncu capture of {rec['captured']} predates the current {rec['source']}: not reported"
    return rec["bytes"], (f"dram__bytes_read.sum + dram__bytes_write.sum of one {rec['kernel']} launch, ncu capture of "
                          f"{rec['captured']} (kernel source sha256 {rec['source_sha256_16']})")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--blocks", type=int, default=15, help="timed blocks of --steps steps; the median block is reported")
    ap.add_argument("--no-side", action="store_true", help="skip the side records (c3, c4, c5_strong, head_sharded, reference_gpu)")
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5", "prefill"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--collective", default="infiniccl", choices=["infiniccl", "torch", "peer"],
                    help="head mode only: the all-gather goes through libinfiniccl.so (default) or torch.distributed; "
                         "peer: no all-gather - the attention kernels store each rank's head slice into every rank's full "
                         "output in symmetric memory, and a barrier follows")
    ap.add_argument("--mode", default="seq", choices=["seq", "head"],
                    help="seq: shard by sequence, no collective (default); head: optional KV-head-sharded mode, "
                         "every rank holds all sequences for its kv-heads and outputs are all-gathered over NCCL")
    ap.add_argument("--cpu-seqs", type=int, default=0, help="sequences in the CPU sample (0 = the whole batch)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-clocks", action="store_true", help="skip nvidia-smi sampling (for short runs under a profiler)")
    return ap.parse_args()


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


WORKLOAD_TEXT = {
    "c2": "configs[1]: Llama-3-8B-shape decode, bf16, batch 64 per GPU, 32/8 heads, head 128, block 16, every seq_len 4096, "
          "permuted tables over a 16384-block pool, 64 new K/V rows cached before attention",
    "c3": "configs[2]: ragged 72B-shape decode, bf16, batch 256, 64/8 heads, head 128, block 16, seq_lens log-uniform [16,32768]",
    "c4": "configs[3]: long-context decode, fp16, batch 2, 32/8 heads, head 128, block 16, seq_lens 131072",
    "c5": "configs[4]: 2048-sequence batch, bf16, 64/8 heads, head 128, seq_lens U[1024,8192], round-robin over the GPUs",
}


def workload_lengths(name, rank=0, world=1, mode="seq"):
    """Sequence lengths one rank holds for a workload (the seeded generators of infinicore_b200.workloads)."""
    import torch

    from infinicore_b200 import workloads

    if name == "c2":
        return torch.full((64,), 4096, dtype=torch.int64)
    if name == "c3":
        return workloads.config3_lengths(seed=3 + (rank if mode == "seq" else 0))
    if name == "c4":
        return torch.full((2,), 131072, dtype=torch.int64)
    lens = workloads.config5_lengths()
    return lens[rank::world] if mode == "seq" else lens


def workload_config(name, n_gpus, mode="seq", collective="infiniccl"):
    """The `config` object of the JSON line: a function of the arguments only, so the GPU arm and the
    reference arm print the same one."""
    lens = workload_lengths(name, 0, n_gpus, mode)
    head_mode = mode == "head" and n_gpus > 1
    kvh = 8 // n_gpus if head_mode else 8
    tokens = int(lens.sum())
    kv_bytes = tokens * kvh * 256 * 2
    return {
        "workload": WORKLOAD_TEXT[name],
        "num_seqs_per_gpu": int(lens.numel()),
        "tokens_per_gpu": tokens,
        "kv_bytes_per_gpu": kv_bytes,
        "parallelism": (f"kv-head-sharded x{n_gpus}, outputs combined per step by {collective}" if head_mode
                        else f"sequence-sharded x{n_gpus}, no collective"),
        "l2": ("inputs larger than L2 (KV working set per step >> 126 MB)" if kv_bytes > (256 << 20)
               else "L2 flushed between steps (a 256 MB buffer is rewritten before every timed step)"),
    }


COLLECTIVE_TEXT = {"infiniccl": "one infinicclAllGather (NCCL)", "torch": "one torch.distributed all-gather (NCCL)",
                   "peer": "peer stores from the attention kernels into every rank's full output + a barrier"}


def make_case(name, rank, world, device, mode="seq"):
    import torch

    from infinicore_b200 import workloads

    if mode == "head" and world > 1:
        # every rank: all sequences, its slice of the kv-heads (and of the q-heads that read them)
        heads, kvh = (32, 8) if name in ("c2", "c4") else (64, 8)
        lens = {"c2": lambda: torch.full((64,), 4096), "c3": workloads.config3_lengths,
                "c4": lambda: torch.full((2,), 131072), "c5": workloads.config5_lengths}[name]()
        assert kvh % world == 0, "kv-heads must divide over the ranks"
        return workloads.build_case(f"{name}_headshard{rank}of{world}", dtype=torch.float16 if name == "c4" else torch.bfloat16,
                                    seq_lens=lens, num_heads=heads // world, num_kv_heads=kvh // world, head_size=128,
                                    block_size=16, seed=7, device=device)

    if name == "c2":
        return workloads.config2_llama8b(seed=2 + rank, device=device)
    if name == "c3":
        return workloads.config3_ragged72b(seed=3 + rank, device=device)
    if name == "c4":
        return workloads.config4_longctx(seed=4 + rank, device=device)
    return workloads.config5_shard(rank, world, device=device)


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle (a port of the reference's torch checker) on all host threads
# ---------------------------------------------------------------------------------------------
def cpu_sample(case_name, num_seqs_cap):
    """A bounded CPU-resident sample of the workload: the first `num_seqs_cap` sequences of it (same
    shapes, lengths and value distribution; pool sized to the sample)."""
    import torch

    from infinicore_b200 import workloads

    if case_name == "c2":
        n = num_seqs_cap or 64
        return workloads.config2_llama8b(seed=2, device="cpu", num_seqs=n), f"{n} of 64 sequences x 4096 tokens"
    if case_name == "c3":
        n = num_seqs_cap or 32
        return workloads.config3_ragged72b(seed=3, device="cpu", num_seqs=n), f"{n} of 256 sequences"
    if case_name == "c4":
        return workloads.config4_longctx(seed=4, device="cpu", num_seqs=1, seq_len=32768), "1 sequence x 32768 of 131072 tokens"
    lens = workloads.config5_lengths()[: (num_seqs_cap or 32)]
    c = workloads.build_case("c5_cpu_sample", dtype=torch.bfloat16, seq_lens=lens, num_heads=64, num_kv_heads=8,
                             head_size=128, block_size=16, seed=5, device="cpu")
    return c, f"{len(lens)} of 2048 sequences"


def run_cpu(case, steps, warmup):
    """Times `steps` passes of caching + attention on the CPU oracle; returns (GB/s, ms/step, threads)."""
    import numpy as np
    import torch

    import oracle

    def bits(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    # all the host threads the process may use, also under a launcher that exports OMP_NUM_THREADS=1
    oracle.use_all_cores()
    code = 12 if case.dtype == torch.float16 else 19
    q, kc, vc = bits(case.q), bits(case.k_cache), bits(case.v_cache)
    nk, nv = bits(case.new_k), bits(case.new_v)
    bt, sl, sm = case.block_tables.numpy(), case.seq_lens.numpy(), case.slot_mapping.numpy()
    out = np.zeros((case.num_seqs, case.num_heads, vc.shape[3]), dtype=np.float64)

    def step():
        oracle.paged_caching(kc, vc, nk, nv, sm)
        oracle.paged_attention(q, kc, vc, bt, sl, case.scale, code, mode="reference", out=out)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return case.kv_bytes / dt / 1e9, dt * 1e3, oracle.num_threads()


def reference_arm(args):
    """The reference's CPU path for this workload (the C/OpenMP port of its torch checker: it has no CPU
    kernel), W warm-up and exactly K timed steps on every host core this process may use.  A step is a
    bounded sample of the workload - the whole batch while K steps of it fit into about two minutes,
    its first n sequences otherwise - and the line says which."""
    import torch

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from infinicore_b200 import workloads  # noqa: F401  (builders used by cpu_sample)

    steps, warmup = max(1, args.steps), max(0, args.warmup)
    case, sample = cpu_sample(args.workload, args.cpu_seqs)
    if not args.cpu_seqs:
        # size the sample from one probe step of the whole batch
        _, probe_ms, _ = run_cpu(case, steps=1, warmup=0)
        budget_ms = 120e3 / (steps + warmup)
        if probe_ms > budget_ms and case.num_seqs > 1:
            n = max(1, int(case.num_seqs * budget_ms / probe_ms))
            case, sample = cpu_sample(args.workload, n)
    gbs, ms, threads = run_cpu(case, steps, warmup)
    full = workload_config(args.workload, args.gpus, args.mode, COLLECTIVE_TEXT[args.collective])
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if args.workload == "c5" else "weak", "vs_baseline": None,
        "dtype": "bf16" if args.workload != "c4" else "f16", "data": "synthetic",
        "config": full,
        "sample": sample + " per step",
        "seqs_per_s": case.num_seqs / (ms / 1e3),
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample + " per step",
                         "processes": 1},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference has no CPU kernel for this path; this is the C/OpenMP port of its torch checker, ONE process on "
                "the host cores whatever --gpus says (a ratio against N GPUs is N GPUs over one CPU process)",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
            return
        # nvidia-smi needs a moment before its first row; do not start timing before it samples
        deadline = time.time() + 3.0
        while time.time() < deadline and os.path.getsize(self.file.name) == 0:
            time.sleep(0.02)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        for row in self.file.read().splitlines():
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


class AbiStep:
    """Descriptors + workspace for one rank's decode step, called through the C ABI on torch's current stream."""

    def __init__(self, case, out=None):
        import torch

        from infinicore_b200.libinfiniop import (LIBINFINIOP, InfiniDeviceEnum, TestTensor, check_error, create_handle,
                                                 infiniopOperatorDescriptor_t, to_infini_dtype)

        self.lib = LIBINFINIOP
        self.check = check_error
        self.case = case
        dev = case.q.device.index
        check_error(LIBINFINIOP.infinirtSetDevice(InfiniDeviceEnum.NVIDIA, dev))
        self.handle = create_handle()
        # `out` given: a (possibly strided) view the descriptor is made for, e.g. this rank's head slice
        # inside its full output in symmetric memory
        self.out = out if out is not None else torch.zeros((case.num_seqs, case.num_heads, case.v_cache.shape[3]), dtype=case.dtype,
                                                            device=case.q.device)

        def tt(t):
            return TestTensor.from_torch(t, to_infini_dtype(t.dtype), InfiniDeviceEnum.NVIDIA)

        a = [tt(self.out), tt(case.q), tt(case.k_cache), tt(case.v_cache), tt(case.block_tables), tt(case.seq_lens)]
        self.attn = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedAttentionDescriptor(self.handle, ctypes.byref(self.attn), *[t.descriptor for t in a], None, case.scale))
        size = ctypes.c_size_t(0)
        check_error(LIBINFINIOP.infiniopGetPagedAttentionWorkspaceSize(self.attn, ctypes.byref(size)))
        self.ws_size = size.value
        self.ws = torch.empty(max(size.value, 1), dtype=torch.uint8, device=case.q.device)
        c = [tt(case.k_cache), tt(case.v_cache), tt(case.new_k), tt(case.new_v), tt(case.slot_mapping)]
        self.cache = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedCachingDescriptor(self.handle, ctypes.byref(self.cache), *[t.descriptor for t in c]))
        # the one-call form of the same step (no reference counterpart): reported beside the two-call step
        f = [tt(self.out), tt(case.q), tt(case.k_cache), tt(case.v_cache), tt(case.new_k), tt(case.new_v), tt(case.block_tables),
             tt(case.seq_lens)]
        self.fused = infiniopOperatorDescriptor_t()
        check_error(LIBINFINIOP.infiniopCreatePagedDecodeStepDescriptor(self.handle, ctypes.byref(self.fused), *[t.descriptor for t in f],
                                                                        None, case.scale))
        for t in a + c + f:
            t.destroy_desc()
        # caching + (streaming path: main + combine, plus a plan launch for batches > 4095 sequences;
        # generic path: one kernel)
        # caching + (reset kernel, [plan kernel for more than 4095 sequences], main kernel, [combine kernel when units * 4 <= workers])
        units = case.num_seqs * case.k_cache.shape[1] * (1 if case.num_heads // case.k_cache.shape[1] <= 8 else -(-(case.num_heads // case.k_cache.shape[1]) // 16))
        combine = 1 if units * 4 <= 148 * 2 * 4 else 0
        reset = 1 - combine  # the counters are only used (and cleared) when the units are merged inside the main kernel
        self.launches_per_step = 1 + ((1 + reset + (0 if case.num_seqs <= 4095 else 1) + combine) if self.ws_size > 0 else 1)

    def caching(self, stream):
        c = self.case
        self.check(self.lib.infiniopPagedCaching(self.cache, None, 0, c.k_cache.data_ptr(), c.v_cache.data_ptr(),
                                                 c.new_k.data_ptr(), c.new_v.data_ptr(), c.slot_mapping.data_ptr(), stream))

    def fused_step(self, stream):
        c = self.case
        self.check(self.lib.infiniopPagedDecodeStep(self.fused, self.ws.data_ptr(), self.ws_size, self.out.data_ptr(), c.q.data_ptr(),
                                                    c.k_cache.data_ptr(), c.v_cache.data_ptr(), c.new_k.data_ptr(), c.new_v.data_ptr(),
                                                    c.block_tables.data_ptr(), c.seq_lens.data_ptr(), None, stream))

    def make_rope(self):
        """Descriptors for a decode layer WITH its rotary embedding: the four calls a caller of the reference
        issues (rope on q, rope on the new K, caching, attention) and the one call that does all of it."""
        import torch

        from infinicore_b200.libinfiniop import InfiniDeviceEnum, TestTensor, infiniopOperatorDescriptor_t, to_infini_dtype

        c = self.case
        dev = c.q.device
        self.pos = (c.seq_lens.to(torch.int64) - 1).clamp(min=0)
        table_len, dhead = int(self.pos.max().item()) + 1, c.q.shape[-1]
        freqs = 1.0 / (1e4 ** (torch.arange(0, dhead, 2, device=dev).float() / dhead))
        angles = torch.outer(torch.arange(table_len, device=dev).float(), freqs)
        self.sin, self.cos = torch.sin(angles).to(c.dtype), torch.cos(angles).to(c.dtype)
        self.q_rot, self.k_rot = torch.empty_like(c.q), torch.empty_like(c.new_k)

        def tt(t):
            return TestTensor.from_torch(t, to_infini_dtype(t.dtype), InfiniDeviceEnum.NVIDIA)

        made = []
        self.rope_q, self.rope_k, self.fused_rope = (infiniopOperatorDescriptor_t() for _ in range(3))
        for desc, y, x in ((self.rope_q, self.q_rot, c.q), (self.rope_k, self.k_rot, c.new_k)):
            t = [tt(y), tt(x), tt(self.pos), tt(self.sin), tt(self.cos)]
            self.check(self.lib.infiniopCreateRoPEDescriptor(self.handle, ctypes.byref(desc), *[d.descriptor for d in t], 1))
            made += t
        f = [tt(self.out), tt(c.q), tt(c.k_cache), tt(c.v_cache), tt(c.new_k), tt(c.new_v), tt(c.block_tables), tt(c.seq_lens)]
        r = [tt(self.pos), tt(self.sin), tt(self.cos)]
        self.check(self.lib.infiniopCreatePagedDecodeStepRoPEDescriptor(
            self.handle, ctypes.byref(self.fused_rope), *[d.descriptor for d in f], None, *[d.descriptor for d in r], 1, c.scale))
        size = ctypes.c_size_t(0)
        self.check(self.lib.infiniopGetPagedDecodeStepWorkspaceSize(self.fused_rope, ctypes.byref(size)))
        self.rope_ws_size = size.value
        self.rope_ws = torch.empty(max(size.value, 1), dtype=torch.uint8, device=dev)
        for d in made + f + r:
            d.destroy_desc()

    def rope_four_calls(self, stream):
        c = self.case
        for desc, y, x in ((self.rope_q, self.q_rot, c.q), (self.rope_k, self.k_rot, c.new_k)):
            self.check(self.lib.infiniopRoPE(desc, None, 0, y.data_ptr(), x.data_ptr(), self.pos.data_ptr(), self.sin.data_ptr(),
                                             self.cos.data_ptr(), stream))
        self.check(self.lib.infiniopPagedCaching(self.cache, None, 0, c.k_cache.data_ptr(), c.v_cache.data_ptr(),
                                                 self.k_rot.data_ptr(), c.new_v.data_ptr(), c.slot_mapping.data_ptr(), stream))
        self.check(self.lib.infiniopPagedAttention(self.attn, self.ws.data_ptr(), self.ws_size, self.out.data_ptr(), self.q_rot.data_ptr(),
                                                   c.k_cache.data_ptr(), c.v_cache.data_ptr(), c.block_tables.data_ptr(),
                                                   c.seq_lens.data_ptr(), None, stream))

    def rope_one_call(self, stream):
        c = self.case
        self.check(self.lib.infiniopPagedDecodeStepRoPE(
            self.fused_rope, self.rope_ws.data_ptr(), self.rope_ws_size, self.out.data_ptr(), c.q.data_ptr(), c.k_cache.data_ptr(),
            c.v_cache.data_ptr(), c.new_k.data_ptr(), c.new_v.data_ptr(), c.block_tables.data_ptr(), c.seq_lens.data_ptr(), None,
            self.pos.data_ptr(), self.sin.data_ptr(), self.cos.data_ptr(), stream))

    def attention_multi_out(self, stream, destinations):
        """Attention with the output rows stored to every destination (tensor or raw address); the first is self.out."""
        c = self.case
        ptrs = [d.data_ptr() if hasattr(d, "data_ptr") else int(d) for d in destinations]
        arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
        self.check(self.lib.infiniopPagedAttentionMultiOut(self.attn, self.ws.data_ptr(), self.ws_size, arr, len(ptrs), c.q.data_ptr(),
                                                          c.k_cache.data_ptr(), c.v_cache.data_ptr(), c.block_tables.data_ptr(),
                                                          c.seq_lens.data_ptr(), None, stream))

    def attention(self, stream):
        c = self.case
        self.check(self.lib.infiniopPagedAttention(self.attn, self.ws.data_ptr(), self.ws_size, self.out.data_ptr(), c.q.data_ptr(),
                                                   c.k_cache.data_ptr(), c.v_cache.data_ptr(), c.block_tables.data_ptr(),
                                                   c.seq_lens.data_ptr(), None, stream))


def gpu_arm(args):
    import torch
    import torch.distributed as dist

    import infinicore_b200 as ib
    from infinicore_b200 import sharding, workloads

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path (use --impl reference for the CPU port)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import datetime

        # a short collective timeout: a rank mismatch should fail in a minute, not hold the GPUs
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=90))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_ranks(values, op):
        """Element-wise reduction of a list of floats over the ranks."""
        if world == 1:
            return list(values)
        t = torch.tensor(list(values), dtype=torch.float64, device=device)
        dist.all_reduce(t, op=op)
        return t.tolist()

    def max_over_ranks(x):
        return reduce_ranks([x], dist.ReduceOp.MAX)[0] if world > 1 else x

    def min_over_ranks(x):
        return reduce_ranks([x], dist.ReduceOp.MIN)[0] if world > 1 else x

    def sum_over_ranks(x):
        return reduce_ranks([x], dist.ReduceOp.SUM)[0] if world > 1 else x

    def all_ranks_ok(ok):
        """True only if every rank reports ok: every rank then takes the same branch (the branches contain
        rank-wide reductions, and sometimes collectives)."""
        return min_over_ranks(1.0 if ok else 0.0) > 0.5

    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream

    def timed(fn, iters):
        """Device time of `iters` back-to-back calls of fn, bracketed by a barrier and a synchronize on
        both sides; nothing but fn's own launches sits between the two events."""
        a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a_ev.record(stream)
        for _ in range(iters):
            fn()
        b_ev.record(stream)
        barrier()
        return a_ev.elapsed_time(b_ev)

    def timed_blocks(fn, iters, blocks):
        """`blocks` timed blocks of `iters` calls; per block the slowest rank's ms per call.  Returns
        (median, min, max, this rank's own median) over the blocks."""
        mine = [timed(fn, iters) / iters for _ in range(blocks)]
        worst = reduce_ranks(mine, dist.ReduceOp.MAX) if world > 1 else mine
        return statistics.median(worst), min(worst), max(worst), statistics.median(mine)

    head_mode = args.mode == "head" and world > 1
    case = make_case(args.workload, rank, world, device, args.mode)
    peers = None
    if head_mode and args.collective == "peer":
        peers = sharding.PeerOutputs(case.num_seqs, case.num_heads * world, case.v_cache.shape[3], case.dtype, device)
    step = AbiStep(case, out=peers.local_slice() if peers is not None else None)
    small_ws = case.kv_bytes <= (256 << 20)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if small_ws else None

    gather_staging = None
    ccl_comm = None  # infinicclAllGather through libinfiniccl.so; None: torch.distributed's all-gather
    if head_mode:
        gather_staging = torch.empty((world, *step.out.shape), dtype=step.out.dtype, device=device)
        if args.collective == "infiniccl":
            from infinicore_b200 import ccl

            ccl_comm = ccl.init_from_process_group()

    def one_step():
        step.caching(sptr)
        if peers is not None:
            # the head slice goes into every rank's full output (two alternating buffers), then one barrier
            step.attention_multi_out(sptr, peers.destinations())
            peers.barrier()
            peers.advance()
        else:
            step.attention(sptr)
            if head_mode:
                sharding.gather_head_sharded(step.out, world, staging=gather_staging, comm=ccl_comm)

    # ---- device-resident timing -------------------------------------------------------------
    W = max(args.warmup, 3)
    K = max(args.steps, 1)
    R = max(args.blocks, 1)
    for _ in range(W):
        one_step()
    barrier()
    sampler = ClockSampler(local_rank)
    sample_clocks = rank == 0 and not args.no_clocks
    if sample_clocks:
        sampler.start()

    if flush is None:
        ms_per_step, ms_min, ms_max, _ = timed_blocks(one_step, K, R)
    else:
        # small working set: scrub L2 before every step and time each step on its own
        per_block = []
        for _ in range(R):
            total = 0.0
            for i in range(K):
                flush.fill_(i & 0xff)
                total += timed(one_step, 1)
            per_block.append(total / K)
        worst = reduce_ranks(per_block, dist.ReduceOp.MAX) if world > 1 else per_block
        ms_per_step, ms_min, ms_max = statistics.median(worst), min(worst), max(worst)
    timed_ms = ms_per_step * K * R
    clock_window = "timed region"
    if not args.no_clocks and timed_ms < 400.0:
        # Too short for nvidia-smi's 100 ms sampling: keep the identical load running (untimed) so the
        # clocks under this load are still observed.  Every rank runs the same number of extra steps
        # (the count derives from the rank-agreed step time), because a step may contain a collective.
        extra = int(600.0 / max(ms_per_step, 1e-3))
        for _ in range(extra):
            one_step()
        torch.cuda.synchronize()
        clock_window = f"timed region ({timed_ms:.1f} ms) + {extra} identical untimed steps"
    clocks = sampler.stop() if sample_clocks else None
    if clocks is not None:
        clocks["window"] = clock_window

    # the dominant kernel on its own: attention calls back to back (plan/combine launches included)
    attn_ms, attn_min, attn_max, _ = timed_blocks(lambda: step.attention(sptr), K, R)
    cache_ms = timed(lambda: step.caching(sptr), K) / K
    fused_ms = None
    if flush is None and not head_mode:
        for _ in range(3):
            step.fused_step(sptr)
        fused_ms = timed_blocks(lambda: step.fused_step(sptr), K, min(R, 5))[0]
    # the same layer with its rotary embedding (q and the new K row rotated first): four calls against one
    rope_ms = None
    if flush is None and not head_mode and case.q.shape[-1] == case.k_cache.shape[-1] and case.q.shape[-1] % 2 == 0:
        # a side measurement: it must never cost the run its headline line
        try:
            step.make_rope()
            for fn in (step.rope_four_calls, step.rope_one_call):
                for _ in range(3):
                    fn(sptr)
            rope_ok = True
        except Exception as exc:  # noqa: BLE001
            print(f"[bench] rope_step skipped on rank {rank}: {exc}", file=sys.stderr)
            rope_ok = False
        if all_ranks_ok(rope_ok):
            rope_ms = (timed_blocks(lambda: step.rope_four_calls(sptr), K, min(R, 5))[0],
                       timed_blocks(lambda: step.rope_one_call(sptr), K, min(R, 5))[0])

    kv_bytes_all = sum_over_ranks(float(case.kv_bytes))
    seqs_all = sum_over_ranks(float(case.num_seqs))
    value = kv_bytes_all / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public Python API, host buffers in and out ---------------------
    # The public call for a whole step: DecodeStep keeps one pinned host arena (q, new K/V rows, slots,
    # block tables, lengths), copies it to the device in one transfer, runs caching + attention and
    # copies the output back, all replayed from one CUDA graph.
    estep = ib.DecodeStep(case.k_cache, case.v_cache, num_seqs=case.num_seqs, num_heads=case.num_heads,
                          max_blocks_per_seq=case.block_tables.shape[1], scale=case.scale)
    for k in ("q", "new_k", "new_v", "slot_mapping", "block_tables", "seq_lens"):
        estep.host[k].copy_(getattr(case, k).cpu())
    estep.capture()  # records both ways of delivering the output (copy node / the kernels' own stores) and keeps the faster
    h2d, d2h = estep.h2d_bytes, estep.d2h_bytes
    e2e_route = {"output_route": "kernels store into pinned host memory" if estep.direct_output else "device-to-host copy node",
                 "chosen_at_capture_from_us": {k: round(v * 1e6, 2) for k, v in getattr(estep, "auto_times", {}).items()}}

    def e2e_step():
        estep.run(sync=True)  # the host reads the step's result before it issues the next step

    if head_mode:
        # NCCL inside the step: issue the calls directly instead of replaying a graph
        host_full = torch.empty((case.num_seqs, case.num_heads * world, step.out.shape[2]), dtype=step.out.dtype).pin_memory()
        d2h = host_full.numel() * host_full.element_size()

        def e2e_step():  # noqa: F811
            estep._dev_arena.copy_(estep._host_arena, non_blocking=True)
            ib.paged_caching(case.k_cache, case.v_cache, estep.dev["new_k"], estep.dev["new_v"], estep.dev["slot_mapping"])
            if peers is not None:
                ib.paged_attention_multi_out(peers.destinations(), estep.dev["q"], case.k_cache, case.v_cache,
                                             estep.dev["block_tables"], estep.dev["seq_lens"], None, case.scale)
                peers.barrier()
                full = peers.full
                peers.advance()
            else:
                o = ib.paged_attention(estep.dev["q"], case.k_cache, case.v_cache, estep.dev["block_tables"], estep.dev["seq_lens"],
                                       None, case.scale, out=estep.out)
                full = sharding.gather_head_sharded(o, world, staging=gather_staging, comm=ccl_comm)
            host_full.copy_(full, non_blocking=True)
            stream.synchronize()

    for _ in range(3):
        e2e_step()
    e2e_ms, e2e_min, e2e_max, _ = timed_blocks(e2e_step, K, R)
    e2e_value = kv_bytes_all / (e2e_ms * 1e-3) / 1e9

    # ---- side records -----------------------------------------------------------------------------
    side = {}
    if not args.no_side and args.workload == "c2" and not head_mode:
        K_side, R_side = min(K, 20), min(R, 5)

        def side_case(build, label):
            """Builds a workload on this rank, times its decode step (caching + attention) like the headline.
            Returns this rank's record or None; never raises."""
            try:
                c = build()
                st = AbiStep(c)

                def fn():
                    st.caching(sptr)
                    st.attention(sptr)

                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                ok = True
            except Exception as exc:  # noqa: BLE001
                print(f"[bench] side record {label} skipped on rank {rank}: {exc}", file=sys.stderr)
                ok, c, fn = False, None, None
            if not all_ranks_ok(ok):
                return None
            med, lo, hi, own = timed_blocks(fn, K_side, R_side)
            attn_only = timed_blocks(lambda: st.attention(sptr), K_side, R_side)[0]
            bytes_all = sum_over_ranks(float(c.kv_bytes))
            rec = {"ms_per_step": med, "ms_min": lo, "ms_max": hi, "value": bytes_all / (med * 1e-3) / 1e9, "unit": UNIT,
                   "attn_ms": attn_only, "num_seqs": int(sum_over_ranks(float(c.num_seqs))),
                   "tokens": int(sum_over_ranks(float(c.total_tokens))), "kv_bytes": int(bytes_all),
                   "seqs_per_s": sum_over_ranks(float(c.num_seqs)) / (med * 1e-3), "steps": K_side, "blocks": R_side,
                   "_own_ms": own, "_own_tokens": float(c.total_tokens)}
            del st, c
            torch.cuda.empty_cache()
            return rec

        peak_now = measured_peak()[0]
        if world == 1:
            for name, build in (("c3", lambda: workloads.config3_ragged72b(seed=3, device=device)),
                                ("c4", lambda: workloads.config4_longctx(seed=4, device=device))):
                rec = side_case(build, name)
                if rec is not None:
                    rec.pop("_own_ms"), rec.pop("_own_tokens")
                    rec["frac"] = rec["kv_bytes"] / (rec["attn_ms"] * 1e-3) / 1e9 / peak_now
                    rec["frac_whole_step"] = rec["value"] / peak_now
                    rec["workload"] = WORKLOAD_TEXT[name]
                side[name] = rec

        # BASELINE configs[4]: ONE batch of 2048 sequences split over the N ranks (strong scaling), each rank
        # with its own pool; two placement policies
        all_lens = workloads.config5_lengths()
        c5 = {"workload": WORKLOAD_TEXT["c5"], "scaling": "strong", "n_gpus": world}
        for policy in (("round_robin",) if world == 1 else ("round_robin", "balanced")):
            idx = sharding.shard(all_lens.tolist(), rank, world, policy)

            def build(idx=idx, policy=policy):
                return workloads.build_case(f"c5_{policy}_{rank}of{world}", dtype=torch.bfloat16, seq_lens=all_lens[idx], num_heads=64,
                                            num_kv_heads=8, head_size=128, block_size=16, max_blocks_per_seq=8192 // 16,
                                            seed=5000 + rank, device=device)

            rec = side_case(build, f"c5_strong/{policy}")
            if rec is not None:
                own_ms, own_tok = rec.pop("_own_ms"), rec.pop("_own_tokens")
                rec["rank_ms_min"] = min_over_ranks(own_ms)
                rec["rank_ms_max"] = max_over_ranks(own_ms)
                rec["rank_tokens_min"] = int(min_over_ranks(own_tok))
                rec["rank_tokens_max"] = int(max_over_ranks(own_tok))
                rec["slowest_rank_token_share"] = rec["rank_tokens_max"] / max(rec["tokens"], 1)
                rec["frac_of_hbm_peak"] = rec["value"] / (peak_now * world)
            c5[policy] = rec
        if world == 1 and c5.get("round_robin") is not None:
            c5["balanced"] = "same as round_robin on one GPU"
        side["c5_strong"] = c5

        # KV-head-sharded mode at N > 1 (configs[4]'s optional variant, on the configs[1] shape): every rank holds all
        # 64 sequences for kv_heads / N of the kv-heads; the outputs are combined (a) by one infinicclAllGather,
        # (b) by the attention kernels' own stores into every rank's full output plus a barrier
        if world > 1 and 8 % world == 0:
            hs = {"workload": "configs[1] shape sharded by kv-head over the ranks (8 / N kv-heads and 32 / N q-heads per rank)"}
            try:
                from infinicore_b200 import ccl

                hcase = make_case("c2", rank, world, device, "head")
                hpeers = sharding.PeerOutputs(hcase.num_seqs, hcase.num_heads * world, hcase.v_cache.shape[3], hcase.dtype, device)
                hstep_a = AbiStep(hcase)
                hstep_p = AbiStep(hcase, out=hpeers.local_slice())
                hstage = torch.empty((world, *hstep_a.out.shape), dtype=hstep_a.out.dtype, device=device)
                hcomm = ccl.init_from_process_group()
                ok = True
            except Exception as exc:  # noqa: BLE001
                print(f"[bench] head_sharded skipped on rank {rank}: {exc}", file=sys.stderr)
                ok = False
            if all_ranks_ok(ok):
                def step_allgather():
                    hstep_a.caching(sptr)
                    hstep_a.attention(sptr)
                    sharding.gather_head_sharded(hstep_a.out, world, staging=hstage, comm=hcomm)

                def step_peer():
                    hstep_p.caching(sptr)
                    hstep_p.attention_multi_out(sptr, hpeers.destinations())
                    hpeers.barrier()
                    hpeers.advance()

                hflush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if hcase.kv_bytes <= (256 << 20) else None

                def timed_steps(fn):
                    for _ in range(3):
                        fn()
                    if hflush is None:
                        return timed_blocks(fn, K_side, R_side)[0]
                    vals = []
                    for i in range(K_side):
                        hflush.fill_(i & 0xff)
                        vals.append(timed(fn, 1))
                    return max_over_ranks(statistics.median(vals))

                bytes_all = sum_over_ranks(float(hcase.kv_bytes))
                for key, fn in (("allgather", step_allgather), ("peer_store", step_peer)):
                    ms = timed_steps(fn)
                    hs[key + "_ms"] = ms
                    hs[key + "_value"] = bytes_all / (ms * 1e-3) / 1e9
                hs["allgather_via"] = "infinicclAllGather (libinfiniccl.so over NCCL)"
                hs["peer_store_via"] = "infiniopPagedAttentionMultiOut into double-buffered symmetric memory + one barrier per step"
                hs["l2"] = "flushed before every timed step" if hflush is not None else "working set larger than L2"
                torch.cuda.synchronize()
                hcomm.destroy()
            else:
                hs = None
            side["head_sharded"] = hs

    # ---- the path's upstream neighbour: infiniopPagedAttentionPrefill (N = 1 only; never costs the run its line) ----
    if not args.no_side and args.workload == "c2" and world == 1:
        try:
            pcase = workloads.prefill_llama8b(device=device)
            pout = torch.empty((pcase.q.shape[0], pcase.num_heads, pcase.head_size), dtype=pcase.dtype, device=device)

            def prefill_call():
                ib.paged_attention_prefill(pcase.q, pcase.k_cache, pcase.v_cache, pcase.block_tables, pcase.seq_lens,
                                           pcase.cum_seq_lens_q, None, pcase.scale, out=pout)

            for _ in range(5):
                prefill_call()
            torch.cuda.synchronize()
            pms = timed_blocks(prefill_call, 50, 5)[0]
            try:
                tpeak, tkind = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"]), "measured"
            except Exception:  # noqa: BLE001
                tpeak, tkind = 1590.0, "fallback"
            ptf = pcase.flops / (pms * 1e-3) / 1e12
            side["prefill"] = {"ms": pms, "tflops": ptf, "frac": ptf / tpeak, "peak": tpeak, "peak_kind": f"of {tkind} (burst bf16 GEMM)",
                               "bound": "tensor", "kernel": "pagedPrefillUmmaKernel (tcgen05 + TMEM)",
                               "workload": "infiniopPagedAttentionPrefill, Llama-3-8B head shape: bf16, 8 prompts x 2048 new tokens, 32/8 heads, "
                                           "head 128, block 16; flops = 4 x heads x head x causal pairs; median of 5 blocks of 50 calls"}
            del pcase, pout
            torch.cuda.empty_cache()
        except Exception as exc:  # noqa: BLE001
            print(f"[bench] prefill side record skipped: {exc}", file=sys.stderr)
            side["prefill"] = None

    # ---- CPU baseline and the reference's own GPU kernels (rank 0, N = 1 only) -------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_case, sample = cpu_sample(args.workload, args.cpu_seqs)
        gbs, ms, threads = run_cpu(sample_case, steps=3, warmup=1)
        cpu = {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample + " per step, 3 timed steps",
               "ms_per_step": ms, "processes": 1}
    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_side and args.workload == "c2":
        ref_gpu = reference_gpu_leg(case, step, sptr, attn_ms, ms_per_step)

    if rank == 0:
        peak, peak_kind = measured_peak()
        achieved = case.kv_bytes / (attn_ms * 1e-3) / 1e9
        traffic, traffic_source = ncu_traffic(args.workload)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "blocks": R,
            "ms_per_step": ms_per_step, "ms_per_step_min": ms_min, "ms_per_step_max": ms_max,
            "timing": f"median of {R} blocks of {K} back-to-back steps (max over ranks per block); min and max block beside it",
            "higher_is_better": True, "scaling": "strong" if (args.workload == "c5" or head_mode) else "weak",
            "vs_baseline": None, "dtype": "f16" if case.dtype == torch.float16 else "bf16", "data": "synthetic",
            "config": workload_config(args.workload, world, args.mode, COLLECTIVE_TEXT[args.collective]),
            "seqs_per_s": seqs_all / (ms_per_step * 1e-3),
            "frac_of_hbm_peak": value / (peak * world),
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": traffic_source, "peak_kind": f"of {peak_kind}",
                "kernel": "pagedDecodeStreamKernel (timed with every launch of the call: events bracket infiniopPagedAttention)",
                "algorithmic_bytes_per_launch": case.kv_bytes, "attn_ms_mean": attn_ms, "attn_ms_min": attn_min,
                "attn_ms_max": attn_max, "caching_ms_mean": cache_ms,
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "ms_per_step_min": e2e_min, "ms_per_step_max": e2e_max, **e2e_route,
                    "note": "q, new K/V rows, slots, block tables and lengths copied in from pinned host memory and the output copied "
                            "back every step, the host waiting for the result before it issues the next step; the KV cache itself "
                            "is device state"},
            "fused_step": (None if fused_ms is None else
                           {"ms_per_step": fused_ms, "value": kv_bytes_all / (fused_ms * 1e-3) / 1e9, "unit": "GB/s",
                            "note": "the same step through infiniopPagedDecodeStep (cache append inside the attention kernel, "
                                    "one launch less); not the reference's call sequence, so not the headline"}),
            "rope_step": (None if rope_ms is None else
                          {"four_calls_ms": rope_ms[0], "one_call_ms": rope_ms[1],
                           "note": "the decode layer with its rotary embedding: infiniopRoPE(q), infiniopRoPE(new K), infiniopPagedCaching, "
                                   "infiniopPagedAttention against infiniopPagedDecodeStepRoPE"}),
            "gpu_launches": step.launches_per_step * K * R,  # inside the timed region that `value` comes from
            "clocks": clocks,
        }
        line.update(side)
        if ref_gpu is not None:
            line["reference_gpu"] = ref_gpu
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if ccl_comm is not None:
        torch.cuda.synchronize()
        ccl_comm.destroy()
    if world > 1:
        dist.destroy_process_group()


def reference_gpu_leg(case, step, sptr, attn_ms, step_ms):
    """The reference's own CUDA kernels (its sources compiled for sm_100a into oracle/_ref) on the same seeded
    configs[1] inputs, in a child process - the two libraries export the same symbols and never share one.
    Returns the record for the JSON line; never raises."""
    import torch

    ref_root = ROOT / "oracle" / "_ref"
    if not (ref_root / "lib" / "libinfiniop.so").is_file():
        return {"unavailable": "oracle/_ref was not built (the reference checkout is needed for that)"}
    try:
        with tempfile.TemporaryDirectory() as tmp:
            out_path = os.path.join(tmp, "ref.pt")
            spec = {"builder": "config2_llama8b", "kwargs": {"seed": 2, "device": "cuda"}, "iters": 20, "warmup": 3}
            env = dict(os.environ)
            env["INFINI_ROOT"] = str(ref_root)
            for k in [k for k in env if k.startswith("INFINIOP_")]:
                env.pop(k)  # the reference's default environment
            res = subprocess.run([sys.executable, str(ROOT / "oracle" / "ref_kernels.py"), json.dumps(spec), out_path],
                                 env=env, capture_output=True, text=True, timeout=600)
            if res.returncode != 0:
                return {"unavailable": "the reference kernels' child process failed: " + (res.stderr or res.stdout)[-300:]}
            ref = torch.load(out_path)
        # this library on the same inputs: the bench's own case has the same seed; one more step so `out` is current
        step.caching(sptr)
        step.attention(sptr)
        torch.cuda.synchronize()
        diff = (step.out.float().cpu() - ref["out"].float()).abs().max().item()
        return {
            "ms_per_call": ref["attn_ms"], "ms_per_step": ref["step_ms"],
            "value": ref["kv_bytes"] / (ref["attn_ms"] * 1e-3) / 1e9, "unit": UNIT,
            "speedup": ref["attn_ms"] / attn_ms, "speedup_whole_step": ref["step_ms"] / step_ms,
            "max_abs_diff": diff,
            "what": "infiniopPagedAttention of the reference's own kernels (default environment: split-KV, 4 splits), compiled "
                    "for sm_100a from its sources, same seeded inputs, 20 calls after 3 warm-up; speedup = its time per call over "
                    "this library's",
        }
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def prefill_arm(args):
    """Secondary benchmark (the path's upstream neighbour): infiniopPagedAttentionPrefill at the
    Llama-3-8B head shape, 8 prompts x 2048 new tokens, bf16.  Tensor-bound: reported in TFLOP/s of
    the causal attention flops against the measured dense bf16 peak."""
    import torch

    import infinicore_b200 as ib
    from infinicore_b200 import workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(0)
    case = workloads.prefill_llama8b(device="cuda")
    out = torch.empty((case.q.shape[0], case.num_heads, case.head_size), dtype=case.dtype, device="cuda")
    stream = torch.cuda.current_stream()

    def call():
        ib.paged_attention_prefill(case.q, case.k_cache, case.v_cache, case.block_tables, case.seq_lens, case.cum_seq_lens_q,
                                   None, case.scale, out=out)

    K = min(args.steps, 200)
    for _ in range(max(args.warmup, 3)):
        call()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    if not args.no_clocks:
        sampler.start()
    a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a_ev.record(stream)
    for _ in range(K):
        call()
    b_ev.record(stream)
    torch.cuda.synchronize()
    ms = a_ev.elapsed_time(b_ev) / K
    clocks = sampler.stop() if not args.no_clocks else None
    peak = 1590.0
    kind = "fallback"
    pth = ROOT / "MEASURED_PEAKS.json"
    if pth.is_file():
        try:
            peak, kind = float(json.loads(pth.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    tflops = case.flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "paged_attn_prefill_throughput", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "prefill, Llama-3-8B head shape: bf16, 8 prompts x 2048 new tokens, 32/8 heads, head 128, block 16 "
                               "(not a BASELINE config: the decode path's upstream neighbour)",
                   "l2": "K/V of one prompt (8 MiB per kv-head group) is re-read from L2 by design; q/out stream once"},
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak, "traffic": None,
                     "peak_kind": f"of {kind}", "kernel": "pagedPrefillUmmaKernel", "algorithmic_flops_per_launch": case.flops},
        "gpu_launches": K, "clocks": clocks,
    }), flush=True)


def main():
    args = parse_args()
    if args.workload == "prefill":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the prefill workload has no CPU reference arm; use the decode workloads"}))
            return
        prefill_arm(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
