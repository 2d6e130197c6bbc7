"""CUDA graphs for decode-only steps.

A step in which every request brings one token launches well over a hundred small kernels; at
that size the launches, not the kernels, bound the step. Such steps are captured once per
(request capacity, block-table width) as a CUDA graph over a batch padded to the capacity, and
replayed: the host then only fills the step's int32 arrays (pinned), copies them, launches the
graph and reads the sampled tokens back. Padded rows belong to a null request that owns the null
page and the null slot, so they touch nothing live. Each graph has its own workspace, batch
buffer and sampler output, so that nothing it points at is ever moved by a later step.
"""
from __future__ import annotations

import gc
import time
import weakref
from typing import Dict, List, Optional, Tuple

import torch

from ..cache.host import host_module
from ..sampling.sampler import Sampler
from .context import StepBuffers, Workspace


class _Captured:
    def __init__(self):
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.buffers: Optional[StepBuffers] = None
        self.tokens: Optional[torch.Tensor] = None
        self.host_tokens: Optional[torch.Tensor] = None
        self.pad_to: Tuple[int, int, int, int] = (0, 0, 0, 0)
        self.kernels = 0  # kernel launches inside the graph
        self.logits: Optional[torch.Tensor] = None
        self.layout = None  # where the step's arrays lie in the batch buffer (host module StepLayout)


class DecodeGraphs:
    BLOCK_BUCKET = 16  # block-table widths are rounded up to this many pages (one graph per width)
    MAX_GRAPHS = 48    # each graph owns its workspace (75 MB at 64 requests of this model): the oldest go first

    def __init__(self, engine):
        # no reference cycle between the engine and its graphs: both then go away when the engine is
        # dropped, not whenever the garbage collector next runs (which may be inside a later capture)
        self._engine = weakref.ref(engine)
        self.captured: Dict[Tuple[int, int], _Captured] = {}
        self.h2d_bytes = self.d2h_bytes = 0  # of the last step (for measurements)
        self.last: Optional[_Captured] = None  # the graph that ran the last step

    @property
    def engine(self):
        eng = self._engine()
        if eng is None:
            raise RuntimeError("the engine of these decode graphs is gone")
        return eng

    def clear(self) -> None:
        self.captured.clear()

    @staticmethod
    def _capacity(n: int) -> int:
        cap = 1
        while cap < n:
            cap *= 2
        return cap

    def _capture(self, cap: int, blocks: int) -> _Captured:
        eng = self.engine
        H = host_module()
        c = _Captured()
        ws = Workspace(eng.device)
        c.buffers = StepBuffers(eng.device, eng.cm.num_groups, eng.cm.page_size, ws)
        sampler = Sampler(eng.ops, eng.device)
        c.pad_to = (cap, cap, cap, blocks)
        page = eng.cm.page_size

        def prepare(entries):
            ctx = c.buffers.prepare(eng.cm, entries, eng.spec.vocab_size, eng.max_pos, c.pad_to)
            # the longest context this graph may meet decides the key splits of attention (the table
            # is rounded up to whole buckets of pages; no position lies beyond the model's limit)
            ctx.max_seq_len, ctx.max_new_tokens, ctx.decode_only = min(blocks * page, eng.max_pos), 1, True
            return ctx

        empty = H.StepEntries()  # only padded rows: every kernel runs on the null request
        side = torch.cuda.Stream(device=eng.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ctx = prepare(empty)
            for _ in range(2):  # sizes every scratch buffer and loads every kernel before the capture
                logits = eng.model.forward(ctx)
                sampler.sample_device(logits, ctx, cap)
                eng.queue_error_check()  # (its pinned word is made here, not inside the capture)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(eng.device)
        ws.frozen = True
        graph = torch.cuda.CUDAGraph()
        before = eng.ops.launches
        # the sampled tokens are written straight into pinned host memory: no copy to enqueue afterwards
        c.host_tokens = torch.zeros(cap, dtype=torch.int32, pin_memory=True)
        # Nothing may free device memory or destroy a graph while the stream is being recorded: a
        # destructor that runs then (say, of an older graph that the collector finds at this moment)
        # invalidates the capture or ends the process. So: collect before, and not during.
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                logits = eng.model.forward(ctx)
                c.tokens = sampler.sample_device(logits, ctx, cap, out=c.host_tokens)
                c.logits = logits  # of the last replay, padded rows included (read by tests)
                eng.queue_error_check()
        finally:
            if gc_was_on:
                gc.enable()
        c.kernels = eng.ops.launches - before
        c.graph = graph
        c.layout = H.StepLayout.make(cap, cap, cap, blocks, eng.cm.num_groups)
        return c

    def _graph_for(self, cap: int, blocks: int) -> _Captured:
        c = self.captured.pop((cap, blocks), None)
        if c is None:
            c = self._capture(cap, blocks)  # about 15 ms
            while len(self.captured) >= self.MAX_GRAPHS:
                torch.cuda.current_stream().synchronize()  # nothing of the oldest graph is still running
                del self.captured[next(iter(self.captured))]
        self.captured[(cap, blocks)] = c  # most recently used last
        return c

    def run(self, entries) -> List[int]:
        """entries: every request brings exactly one token and wants its logits."""
        eng = self.engine
        H = host_module()
        tokens, seqs, rows, blocks = H.step_caps(eng.cm, entries)
        cap = self._capacity(seqs)
        blocks = (blocks + self.BLOCK_BUCKET - 1) // self.BLOCK_BUCKET * self.BLOCK_BUCKET
        c = self._graph_for(cap, blocks)
        c.buffers.refill(eng.cm, entries, c.layout, eng.spec.vocab_size, eng.max_pos)
        c.graph.replay()
        eng.ops.launches += c.kernels
        t0 = time.perf_counter()
        torch.cuda.current_stream().synchronize()
        eng.sampler.wait_seconds += time.perf_counter() - t0
        eng.raise_if_kernel_error()
        self.h2d_bytes, self.d2h_bytes = c.buffers.h2d_bytes, 4 * cap
        self.last = c
        return c.host_tokens.tolist()[:seqs]

    def run_device(self, entries) -> torch.Tensor:
        """As run, without reading the tokens back (for device-time measurements)."""
        eng = self.engine
        H = host_module()
        tokens, seqs, rows, blocks = H.step_caps(eng.cm, entries)
        cap = self._capacity(seqs)
        blocks = (blocks + self.BLOCK_BUCKET - 1) // self.BLOCK_BUCKET * self.BLOCK_BUCKET
        c = self._graph_for(cap, blocks)
        c.buffers.refill(eng.cm, entries, c.layout, eng.spec.vocab_size, eng.max_pos)
        c.graph.replay()
        eng.ops.launches += c.kernels
        return c.tokens[:seqs]
