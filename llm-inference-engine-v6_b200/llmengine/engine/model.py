"""A model built from its description: embedding, the layers in their run order, final norm, head.

`Model.forward(ctx)` is the device half of the step function: it runs exactly the tokens of the
step's flat batch, reading and writing the paged cache through the block tables in `ctx`, and
returns float32 logits for the wanted rows only (the reference skips the final norm and the head
for positions whose logits are not asked for, src/engine.cpp:415-433).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from ..cache.storage import allocate_run_caches, bytes_per_token, plan_groups
from ..parts.base import BuildEnv, LayerCache, Residual
from ..parts.registry import build_part
from ..parts.spec import ModelSpec
from ..weights.loader import Checkpoint, load_tensors
from ..weights.random_init import model_tensor_needs


class Model:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec, self.env = spec, env
        self.embedding = build_part("embedding", spec.embedding, env)
        self.blocks = [build_part("block", b, env) for b in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, env)
        self.head = build_part("head", spec.head, env)
        n_runs = len(spec.order)
        for r, run in enumerate(spec.order):
            if not (0 <= run.layer < len(self.blocks)):
                raise ValueError(f"layer order entry {r} names layer {run.layer}, which does not exist")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < r):
                    raise ValueError(f"layer order entry {r} reads the cache of entry {run.cache_from}, which must come before it")
                if spec.order[run.cache_from].cache_from is not None:
                    raise ValueError(f"layer order entry {r} reads the cache of entry {run.cache_from}, which owns none")
        # cache needs per run: a run that borrows another run's cache needs nothing of its own
        self.run_needs: List[Sequence[object]] = [
            () if run.cache_from is not None else tuple(self.blocks[run.layer].cache_needs()) for run in spec.order]
        self.windows, self.run_group = plan_groups(self.run_needs)
        # where the scheduler may cut a prompt: the least common multiple of what the layers ask for
        self.portion_multiple = 1
        for needs in self.run_needs:
            for need in needs:
                m = int(getattr(need, "portion_multiple", 1))
                if m < 1:
                    raise ValueError(f"cache need {need!r}: portion_multiple must be >= 1")
                self.portion_multiple = math.lcm(self.portion_multiple, m)
        self.caches: List[LayerCache] = [LayerCache() for _ in range(n_runs)]
        self.weight_bytes = 0

    # ------------------------------------------------------------------ weights
    def load(self, model_dir: str) -> None:
        needs = model_tensor_needs(self.spec)
        tensors = load_tensors(Checkpoint(model_dir), needs, self.spec.duplicates, self.env.device, self.env.dtype,
                               ignore=self.spec.ignore)
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            part.load(tensors)
        self.weight_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
        self.tensor_names = sorted(tensors)

    # ------------------------------------------------------------------ cache
    def kv_bytes_per_token(self) -> int:
        return bytes_per_token(self.run_needs, self.env.dtype)

    def allocate_cache(self, group_pages: Sequence[int], num_slots: int) -> None:
        own = allocate_run_caches(self.run_needs, self.run_group, group_pages, self.windows, self.env.page_size,
                                  num_slots, self.env.dtype, self.env.device)
        for r, run in enumerate(self.spec.order):
            if run.cache_from is None:
                self.caches[r] = own[r]
            else:
                src = own[run.cache_from]
                self.caches[r] = LayerCache(group=src.group, k=src.k, v=src.v, writes=False, window=src.window,
                                            states=src.states)

    def reset_slot(self, slot: int) -> None:
        """A request starts in this slot: its fixed-size state begins at zero."""
        for c in self.caches:
            if c.writes:
                for t in c.states.values():
                    t[slot].zero_()

    # ------------------------------------------------------------------ forward
    def parts(self):
        """Every part of the model, the parts of parts included."""
        todo = [self.embedding, *self.blocks, self.final_norm, self.head]
        while todo:
            part = todo.pop()
            yield part
            todo.extend(part.subparts())

    @property
    def capturable(self) -> bool:
        """Whether a decode step of this model may be recorded as a CUDA graph: every part says so."""
        return all(p.capturable for p in self.parts())

    def kernel_notes(self) -> List[str]:
        seen, out = set(), []
        for p in self.parts():
            for line in p.kernel_notes():
                if line not in seen:
                    seen.add(line)
                    out.append(line)
        return sorted(out)

    def forward(self, ctx) -> torch.Tensor:
        order = self.spec.order
        ctx.stream_sumsq = ctx.stream_prescaled = None
        # who reads the residual stream next: a part that writes it may leave that norm's input prepared
        ctx.next_norm = self.blocks[order[0].layer].first_norm() if order else self.final_norm
        res = Residual(self.embedding.forward(ctx))
        res.sumsq, ctx.stream_sumsq = ctx.stream_sumsq, None
        if ctx.stream_prescaled is not None:
            (res.prescaled, res.prescaled_weight), ctx.stream_prescaled = ctx.stream_prescaled, None
        for r, run in enumerate(order):
            ctx.norm_after_block = self.blocks[order[r + 1].layer].first_norm() if r + 1 < len(order) else self.final_norm
            res = self.blocks[run.layer].forward(res, ctx, self.caches[r])
        ctx.next_norm = ctx.norm_after_block = None
        if ctx.n_rows > 0:
            if self.final_norm.can_defer and self.head.wants_lazy_norm(ctx):
                x = self.final_norm.forward(res, ctx, rows=ctx.logit_rows, n_rows=ctx.n_rows, lazy=True)
            else:
                x = self.final_norm.forward(res, ctx, rows=ctx.logit_rows, n_rows=ctx.n_rows)
        else:
            x = ctx.ws.get("norm.rows_out", (1, self.spec.hidden_size), self.env.dtype)[:0]
        return self.head.forward(x, ctx)
