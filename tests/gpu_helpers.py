"""Helpers of the GPU tests: a step context built the way the engine builds it, for parts run alone."""
from __future__ import annotations

import torch

from llmengine.cache import host_module
from llmengine.engine.context import StepBuffers, Workspace
from llmengine.ops import get_ops
from llmengine.parts.base import BuildEnv, LayerCache

DEV = torch.device("cuda:0")


class Harness:
    """A cache manager, step buffers and one layer's cache, without any model."""

    def __init__(self, dtype, page=4, pages=64, windows=(0,), slots=4, nkv=1, hd=16):
        self.H = host_module()
        self.env = BuildEnv(device=DEV, dtype=dtype, ops=get_ops(), page_size=page)
        self.cm = self.H.CacheManager(page, [self.H.GroupSpec(pages, w) for w in windows], slots)
        self.ws = Workspace(DEV)
        self.buffers = StepBuffers(DEV, len(windows), page, self.ws)
        self.cache = LayerCache(group=0, window=windows[0],
                                k=torch.zeros(pages + 1, nkv, page, hd, dtype=dtype, device=DEV),
                                v=torch.zeros(pages + 1, nkv, page, hd, dtype=dtype, device=DEV))

    def ctx(self, batch, vocab=1 << 30, max_pos=1 << 20):
        """batch: [(request id, n tokens or token list, wanted places)]; reserves and advances."""
        e = self.H.StepEntries()
        for rid, toks, want in batch:
            toks = [0] * toks if isinstance(toks, int) else list(toks)
            if not self.cm.has_request(rid):
                assert self.cm.add_request(rid) >= 0
            assert self.cm.reserve(rid, len(toks))
            e.add(rid, toks, list(want))
        c = self.buffers.prepare(self.cm, e, vocab, max_pos)
        for rid, toks, _ in batch:
            self.cm.advance(rid, toks if isinstance(toks, int) else len(toks))
        return c
