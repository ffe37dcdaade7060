"""TEST / BASELINE INFRASTRUCTURE - times the REFERENCE'S OWN CUDA kernels for the decode step.

Runs in a process of its own with INFINI_ROOT pointing at oracle/_ref (the reference's sources for this
path, compiled for sm_100a by oracle/build_ref.py), because that library exports the same symbols as
this repository's and the two must never share a process.  The decode problem is rebuilt from a seeded
workload spec, so nothing large crosses the process boundary:

    INFINI_ROOT=oracle/_ref python oracle/ref_kernels.py '<json spec>' out.pt

spec = {"builder": "<function in infinicore_b200.workloads>", "kwargs": {...}, "iters": N, "warmup": W}
out.pt = {"out": attention output (cpu), "attn_ms": mean device time of one infiniopPagedAttention call,
          "step_ms": mean device time of infiniopPagedCaching + infiniopPagedAttention, "library": path,
          "kv_bytes": algorithmic KV bytes of one call}

Reference entry points exercised: include/infiniop/ops/paged_attention.h:33-91, paged_caching.h:24-75
(kernels src/infiniop/ops/paged_attention/nvidia/paged_attention_hd128.cu:423-923,
src/infiniop/ops/paged_caching/cuda/kernel.cuh:22-89), default environment.
"""
import ctypes
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    spec = json.loads(sys.argv[1])
    out_path = sys.argv[2]
    from infinicore_b200 import workloads
    from infinicore_b200.libinfiniop import (LIBINFINIOP, InfiniDeviceEnum, TestTensor, check_error, create_handle,
                                             infiniopOperatorDescriptor_t, library_paths, to_infini_dtype)

    kwargs = dict(spec.get("kwargs", {}))
    if "dtype" in kwargs:
        kwargs["dtype"] = getattr(torch, kwargs["dtype"])
    d = getattr(workloads, spec["builder"])(**kwargs).to("cuda")
    check_error(LIBINFINIOP.infinirtSetDevice(InfiniDeviceEnum.NVIDIA, 0))
    handle = create_handle()
    out = torch.zeros((d.num_seqs, d.num_heads, d.v_cache.shape[3]), dtype=d.dtype, device="cuda")

    def tt(t):
        return TestTensor.from_torch(t, to_infini_dtype(t.dtype), InfiniDeviceEnum.NVIDIA)

    a = [tt(out), tt(d.q), tt(d.k_cache), tt(d.v_cache), tt(d.block_tables), tt(d.seq_lens)]
    attn = infiniopOperatorDescriptor_t()
    check_error(LIBINFINIOP.infiniopCreatePagedAttentionDescriptor(handle, ctypes.byref(attn), *[t.descriptor for t in a], None, d.scale))
    size = ctypes.c_size_t(0)
    check_error(LIBINFINIOP.infiniopGetPagedAttentionWorkspaceSize(attn, ctypes.byref(size)))
    ws = torch.ones(max(size.value, 1), dtype=torch.uint8, device="cuda")
    c = [tt(d.k_cache), tt(d.v_cache), tt(d.new_k), tt(d.new_v), tt(d.slot_mapping)]
    cache = infiniopOperatorDescriptor_t()
    check_error(LIBINFINIOP.infiniopCreatePagedCachingDescriptor(handle, ctypes.byref(cache), *[t.descriptor for t in c]))
    for t in a + c:
        t.destroy_desc()
    stream = torch.cuda.current_stream().cuda_stream

    def caching():
        check_error(LIBINFINIOP.infiniopPagedCaching(cache, None, 0, d.k_cache.data_ptr(), d.v_cache.data_ptr(), d.new_k.data_ptr(),
                                                     d.new_v.data_ptr(), d.slot_mapping.data_ptr(), stream))

    def attention():
        check_error(LIBINFINIOP.infiniopPagedAttention(attn, ws.data_ptr(), size.value, out.data_ptr(), d.q.data_ptr(), d.k_cache.data_ptr(),
                                                       d.v_cache.data_ptr(), d.block_tables.data_ptr(), d.seq_lens.data_ptr(), None, stream))

    def timed(fn, iters):
        a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a_ev.record()
        for _ in range(iters):
            fn()
        b_ev.record()
        torch.cuda.synchronize()
        return a_ev.elapsed_time(b_ev) / iters

    def step():
        caching()
        attention()

    for _ in range(max(int(spec.get("warmup", 3)), 1)):
        step()
    iters = max(int(spec.get("iters", 20)), 1)
    result = {"step_ms": timed(step, iters), "attn_ms": timed(attention, iters), "out": out.cpu(),
              "library": str(library_paths()[1]), "kv_bytes": d.kv_bytes, "workspace": size.value}
    check_error(LIBINFINIOP.infiniopDestroyPagedAttentionDescriptor(attn))
    check_error(LIBINFINIOP.infiniopDestroyPagedCachingDescriptor(cache))
    torch.save(result, out_path)


if __name__ == "__main__":
    main()
