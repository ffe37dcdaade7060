"""A whole decode step as one replayable CUDA graph.

The reference's infinicore layer records operators and replays them as CUDA graphs
(src/infinicore/graph/graph.cc:97-171: warm up, capture the capture-safe segment, replay).  This is
the same idea for the one segment this library owns: copy the step's small inputs from pinned host
memory, scatter the new K/V rows into the paged pools (paged_caching), attend (paged_attention),
copy the output back.  Capturing it once removes the per-step host work of five API calls; the
operators themselves allocate nothing and never synchronise, which is what makes them capturable.

    step = DecodeStep(k_cache, v_cache, num_seqs=64, num_heads=32, max_blocks_per_seq=256, scale=s)
    step.host["q"][...] = ...            # fill the pinned inputs: q, new_k, new_v, slot_mapping,
    out = step.run()                     #   block_tables, seq_lens; run() returns the pinned output

The output can travel two ways: a device-to-host copy node after the kernels, or the kernels storing their
rows straight into the pinned buffer over PCIe (direct_output).  Which is faster depends on the machine (the
direct stores ride on the kernel's tail, the copy node is a separate 10 us step): by default capture() records
both, times a few replays of each and keeps the faster.
"""
from __future__ import annotations

import torch

from . import ops

_INPUTS = ("q", "new_k", "new_v", "slot_mapping", "block_tables", "seq_lens")


class DecodeStep:
    def __init__(self, k_cache: torch.Tensor, v_cache: torch.Tensor, *, num_seqs: int, num_heads: int,
                 max_blocks_per_seq: int, scale: float, index_dtype: torch.dtype = torch.int64,
                 alibi_slopes: torch.Tensor | None = None, direct_output: bool | str = "auto"):
        if not (k_cache.is_cuda and v_cache.is_cuda):
            raise RuntimeError("DecodeStep needs the cache pools on a GPU; there is no CPU fallback")
        self.k_cache, self.v_cache = k_cache, v_cache
        self.scale = float(scale)
        self.alibi = alibi_slopes
        self.device = k_cache.device
        _, kvh, _, hd = k_cache.shape
        vd = v_cache.shape[3]
        dt = k_cache.dtype
        layout = {
            "q": ((num_seqs, num_heads, hd), dt),
            "new_k": ((num_seqs, kvh, hd), dt),
            "new_v": ((num_seqs, kvh, vd), dt),
            "slot_mapping": ((num_seqs,), torch.int64),
            "block_tables": ((num_seqs, max_blocks_per_seq), index_dtype),
            "seq_lens": ((num_seqs,), index_dtype),
        }
        offsets, cursor = {}, 0
        for name in _INPUTS:
            shape, dtype = layout[name]
            nbytes = torch.empty((), dtype=dtype).element_size()
            for s in shape:
                nbytes *= s
            offsets[name] = (cursor, nbytes, shape, dtype)
            cursor += (nbytes + 255) // 256 * 256
        self.h2d_bytes = cursor
        self._host_arena = torch.empty(cursor, dtype=torch.uint8).pin_memory()
        self._dev_arena = torch.empty(cursor, dtype=torch.uint8, device=self.device)

        def views(arena):
            return {n: arena[o:o + b].view(d).view(s) for n, (o, b, s, d) in offsets.items()}

        self.host = views(self._host_arena)   # fill these before run()
        self.dev = views(self._dev_arena)
        self.out = torch.empty((num_seqs, num_heads, vd), dtype=dt, device=self.device)
        self.host_out = torch.empty((num_seqs, num_heads, vd), dtype=dt).pin_memory()
        self.d2h_bytes = self.host_out.numel() * self.host_out.element_size()
        # direct_output: the attention kernels store their rows straight into the pinned host buffer (mapped
        # into the device's address space) while they run, instead of a device buffer that is copied afterwards
        # True / False, or "auto": decided by capture()
        self.direct_output = direct_output if direct_output == "auto" else bool(direct_output)
        self._graph = None
        self._stream = torch.cuda.Stream(device=self.device)

    def _issue(self, direct: bool):
        self._dev_arena.copy_(self._host_arena, non_blocking=True)
        ops.paged_caching(self.k_cache, self.v_cache, self.dev["new_k"], self.dev["new_v"], self.dev["slot_mapping"])
        ops.paged_attention(self.dev["q"], self.k_cache, self.v_cache, self.dev["block_tables"], self.dev["seq_lens"],
                            self.alibi, self.scale, out=self.host_out if direct else self.out)
        if not direct:
            self.host_out.copy_(self.out, non_blocking=True)

    def _record(self, direct: bool):
        """Warm up (creates descriptors and the workspace outside the capture), then record the step."""
        with torch.cuda.stream(self._stream):
            for _ in range(3):
                self._issue(direct)
            self._stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self._stream):
                self._issue(direct)
        return graph

    def _time(self, graph, replays: int = 30) -> float:
        """Host time per replay-and-wait of a recorded step, in seconds: what a caller of run() sees."""
        import time

        with torch.cuda.stream(self._stream):
            for _ in range(5):
                graph.replay()
                self._stream.synchronize()
            t0 = time.perf_counter()
            for _ in range(replays):
                graph.replay()
                self._stream.synchronize()
            return (time.perf_counter() - t0) / replays

    def capture(self):
        """Records the step.  With direct_output="auto" both ways of delivering the output are recorded and
        timed on whatever the pinned inputs hold now (fill them with a representative step first; the cache
        rows of that step are written, as by any run()), and the faster one is kept; `direct_output` then
        says which."""
        if self.direct_output == "auto":
            graphs = {d: self._record(d) for d in (False, True)}
            times = {d: self._time(g) for d, g in graphs.items()}
            self.direct_output = times[True] < times[False]
            self.auto_times = {"copy_node_s": times[False], "direct_store_s": times[True]}
            self._graph = graphs[self.direct_output]
        else:
            self._graph = self._record(self.direct_output)
        return self

    def run(self, sync: bool = True) -> torch.Tensor:
        """Replays the captured step with whatever the pinned inputs hold now; returns the pinned
        output (valid once the replay has completed - immediately when sync=True)."""
        if self._graph is None:
            self.capture()
        self._graph.replay()
        if sync:
            # replay() enqueues on the current stream
            torch.cuda.current_stream(self.device).synchronize()
        return self.host_out
