"""Runs one decode step (paged_caching, then paged_attention), one prefill call or one rotary
embedding through the C ABI of whichever libinfiniop the loader finds, in a process of its own.

Used with INFINI_ROOT=oracle/_ref (the reference's own CUDA sources compiled for sm_100a by
oracle/build_ref.py) to obtain the REFERENCE KERNELS' results and timings on identical seeded
inputs, without ever loading both libraries into one process (they export the same symbols).

    INFINI_ROOT=... python tests/ref_runner.py '<json spec>' out.pt

spec = {"builder": "<function in infinicore_b200.workloads>", "kwargs": {...}, "iters": N}
The inputs are rebuilt from the spec (seeded), so nothing large crosses the process boundary.
"""
import json
import os
import statistics
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def run_prefill(spec, case, d, out_path):
    import ctypes

    import abi
    from infinicore_b200.libinfiniop import LIBINFINIOP, InfiniDeviceEnum, TestWorkspace, check_error, library_paths

    out = torch.zeros((d.q.shape[0], d.num_heads, d.v_cache.shape[3]), dtype=d.dtype, device="cuda")
    status, desc = abi.create_prefill(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, d.cum_seq_lens_q, None, d.scale,
                                      path=os.environ.get("INFINIOP_PAGED_PREFILL_PATH"))
    check_error(status)
    size = ctypes.c_size_t(0)
    check_error(LIBINFINIOP.infiniopGetPagedAttentionPrefillWorkspaceSize(desc, ctypes.byref(size)))
    ws = TestWorkspace(size.value, InfiniDeviceEnum.NVIDIA)

    def call(stream=None):
        check_error(LIBINFINIOP.infiniopPagedAttentionPrefill(
            desc, ws.data(), size.value, out.data_ptr(), d.q.data_ptr(), d.k_cache.data_ptr(), d.v_cache.data_ptr(),
            d.block_tables.data_ptr(), d.seq_lens.data_ptr(), d.cum_seq_lens_q.data_ptr(), None, stream))

    call()
    torch.cuda.synchronize()
    result = {"out": out.cpu(), "library": str(library_paths()[1]), "workspace": size.value}
    iters = int(spec.get("iters", 0))
    if iters:
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            call(stream)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            call(stream)
        b.record()
        torch.cuda.synchronize()
        result["attn_ms"] = a.elapsed_time(b) / iters
        result["flops"] = case.flops
    check_error(LIBINFINIOP.infiniopDestroyPagedAttentionPrefillDescriptor(desc))
    torch.save(result, out_path)


def run_rope(spec, out_path):
    """spec = {"op": "rope", "shape": [...], "dtype": "...", "algo": 0 | 1, "seed": n, "table_len": n, "iters": N}"""
    import ctypes

    import abi
    from infinicore_b200.libinfiniop import LIBINFINIOP, check_error, library_paths

    dtype = getattr(torch, spec["dtype"])
    gen = torch.Generator().manual_seed(int(spec.get("seed", 0)))
    shape = list(spec["shape"])
    x = torch.randn(shape, generator=gen).to(dtype).cuda()
    table_len, dhead = int(spec["table_len"]), shape[-1]
    pos = torch.randint(0, table_len, (shape[-3],), generator=gen).cuda()
    freqs = 1.0 / (1e4 ** (torch.arange(0, dhead, 2).float() / dhead))
    angles = torch.outer(torch.arange(table_len).float(), freqs)
    sin, cos = torch.sin(angles).to(dtype).cuda(), torch.cos(angles).to(dtype).cuda()
    y = torch.zeros_like(x)
    status, desc = abi.rope_create(y, x, pos, sin, cos, int(spec["algo"]))
    check_error(status)

    def call(stream=None):
        check_error(LIBINFINIOP.infiniopRoPE(desc, None, 0, y.data_ptr(), x.data_ptr(), pos.data_ptr(), sin.data_ptr(), cos.data_ptr(), stream))

    call()
    torch.cuda.synchronize()
    result = {"y": y.cpu(), "library": str(library_paths()[1])}
    iters = int(spec.get("iters", 0))
    if iters:
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            call(stream)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            call(stream)
        b.record()
        torch.cuda.synchronize()
        result["ms"] = a.elapsed_time(b) / iters
        result["bytes"] = 2 * x.numel() * x.element_size()
    check_error(LIBINFINIOP.infiniopDestroyRoPEDescriptor(desc))
    torch.save(result, out_path)


def run_kv_caching(spec, out_path):
    """spec = {"op": "kv_caching", "shape": [batch, heads, max_len, hidden], "seq_len": n, "dtype": "...", "seed": n, "iters": N}"""
    import abi
    from infinicore_b200.libinfiniop import LIBINFINIOP, check_error, library_paths

    dtype = getattr(torch, spec["dtype"])
    gen = torch.Generator().manual_seed(int(spec.get("seed", 0)))
    shape, seq_len = list(spec["shape"]), int(spec["seq_len"])
    k_cache, v_cache = torch.randn(shape, generator=gen).to(dtype).cuda(), torch.randn(shape, generator=gen).to(dtype).cuda()
    new_shape = [shape[0], shape[1], seq_len, shape[3]]
    k, v = torch.randn(new_shape, generator=gen).to(dtype).cuda(), torch.randn(new_shape, generator=gen).to(dtype).cuda()
    past = torch.randint(0, shape[2] - seq_len + 1, (shape[0],), generator=gen).cuda()
    status, desc = abi.kv_caching_create(k_cache, v_cache, k, v, past)
    check_error(status)

    def call(stream=None):
        check_error(LIBINFINIOP.infiniopKVCaching(desc, None, 0, k_cache.data_ptr(), v_cache.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                  past.data_ptr(), stream))

    call()
    torch.cuda.synchronize()
    result = {"k_cache": k_cache.cpu(), "v_cache": v_cache.cpu(), "library": str(library_paths()[1])}
    iters = int(spec.get("iters", 0))
    if iters:
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            call(stream)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            call(stream)
        b.record()
        torch.cuda.synchronize()
        result["ms"] = a.elapsed_time(b) / iters
        result["bytes"] = 2 * 2 * k.numel() * k.element_size()  # K and V rows, read once and written once
    check_error(LIBINFINIOP.infiniopDestroyKVCachingDescriptor(desc))
    torch.save(result, out_path)


def run_paged_caching(spec, out_path):
    """spec = {"op": "paged_caching", "tokens": n, "kv_heads": h, "head": d, "block": b, "dtype": "...", "seed": n, "iters": N}:
    a prefill-sized scatter (every slot of the pool written once, in shuffled order)."""
    import ctypes

    import abi
    from infinicore_b200.libinfiniop import LIBINFINIOP, check_error, library_paths

    dtype = getattr(torch, spec["dtype"])
    gen = torch.Generator().manual_seed(int(spec.get("seed", 0)))
    tokens, kvh, hd, bs = int(spec["tokens"]), int(spec["kv_heads"]), int(spec["head"]), int(spec["block"])
    blocks = (tokens + bs - 1) // bs
    k_cache = torch.zeros((blocks, kvh, bs, hd), dtype=dtype, device="cuda")
    v_cache = torch.zeros((blocks, kvh, bs, hd), dtype=dtype, device="cuda")
    k, v = torch.randn((tokens, kvh, hd), generator=gen).to(dtype).cuda(), torch.randn((tokens, kvh, hd), generator=gen).to(dtype).cuda()
    # tokens of a prompt land in consecutive slots of shuffled blocks, as a block table would place them
    order = torch.randperm(blocks, generator=gen)
    slots = (order.repeat_interleave(bs) * bs + torch.arange(bs).repeat(blocks))[:tokens].to(torch.int64).cuda()
    status, desc = abi.create_caching(k_cache, v_cache, k, v, slots)
    check_error(status)

    def call(stream=None):
        check_error(LIBINFINIOP.infiniopPagedCaching(desc, None, 0, k_cache.data_ptr(), v_cache.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                     slots.data_ptr(), stream))

    call()
    torch.cuda.synchronize()
    result = {"k_cache": k_cache.cpu(), "v_cache": v_cache.cpu(), "library": str(library_paths()[1])}
    iters = int(spec.get("iters", 0))
    if iters:
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            call(stream)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            call(stream)
        b.record()
        torch.cuda.synchronize()
        result["ms"] = a.elapsed_time(b) / iters
        result["bytes"] = 2 * 2 * k.numel() * k.element_size()
    check_error(LIBINFINIOP.infiniopDestroyPagedCachingDescriptor(desc))
    torch.save(result, out_path)


def main():
    spec = json.loads(sys.argv[1])
    out_path = sys.argv[2]
    if spec.get("op") == "paged_caching":
        return run_paged_caching(spec, out_path)
    if spec.get("op") == "rope":
        return run_rope(spec, out_path)
    if spec.get("op") == "kv_caching":
        return run_kv_caching(spec, out_path)
    from infinicore_b200 import workloads
    from infinicore_b200.libinfiniop import LIBINFINIOP, check_error, library_paths

    import abi

    kwargs = dict(spec.get("kwargs", {}))
    if "dtype" in kwargs:
        kwargs["dtype"] = getattr(torch, kwargs["dtype"])
    case = getattr(workloads, spec["builder"])(**kwargs)
    d = case.to("cuda")
    if isinstance(case, workloads.PrefillCase):
        return run_prefill(spec, case, d, out_path)
    out = torch.zeros((d.num_seqs, d.num_heads, d.v_cache.shape[3]), dtype=d.dtype, device="cuda")
    if spec.get("caching", True):
        abi.paged_caching(d.k_cache, d.v_cache, d.new_k, d.new_v, d.slot_mapping)
    op = abi.AttentionOp(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, None, d.scale)
    check_error(op.status)
    check_error(op.run(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens))
    torch.cuda.synchronize()
    result = {"out": out.cpu(), "library": str(library_paths()[1]), "workspace": op.workspace_size}
    if spec.get("return_cache", False):
        result["k_cache"] = d.k_cache.cpu()
        result["v_cache"] = d.v_cache.cpu()

    iters = int(spec.get("iters", 0))
    if iters:
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(5):
            check_error(op.run(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, stream=stream))
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            check_error(op.run(out, d.q, d.k_cache, d.v_cache, d.block_tables, d.seq_lens, stream=stream))
        b.record()
        torch.cuda.synchronize()
        result["attn_ms"] = a.elapsed_time(b) / iters
        result["kv_bytes"] = case.kv_bytes
    op.destroy()
    torch.save(result, out_path)


if __name__ == "__main__":
    main()
