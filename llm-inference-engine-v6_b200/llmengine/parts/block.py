"""Arrangement of parts in a layer. "pre_norm": h += mixer(norm1(h)); h += feed_forward(norm2(h))
(src/engine.cpp:307-413). The residual sums are fused into the norm that follows them."""
from __future__ import annotations

from typing import List

from .base import Block, LayerCache, Residual
from .registry import build_part, part_class, register_part
from .spec import BlockSpec, TensorNeed


class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec, env):
        super().__init__(spec, env)
        self.norm1 = build_part("norm", spec.norm1, env)
        self.mixer = build_part("mixer", spec.mixer, env)
        self.norm2 = build_part("norm", spec.norm2, env)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, env)

    @staticmethod
    def tensor_needs(spec: BlockSpec) -> List[TensorNeed]:
        out: List[TensorNeed] = []
        for cat, sub in (("norm", spec.norm1), ("mixer", spec.mixer), ("norm", spec.norm2),
                         ("feed_forward", spec.feed_forward)):
            out += part_class(cat, sub.kind).tensor_needs(sub)
        return out

    def subparts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def load(self, tensors) -> None:
        for p in (self.norm1, self.mixer, self.norm2, self.feed_forward):
            p.load(tensors)

    def first_norm(self):
        return self.norm1

    def forward(self, res: Residual, ctx, cache: LayerCache) -> Residual:
        ctx.residual = res  # a part whose last product can add into the stream itself returns None
        x = self._norm(self.norm1, self.mixer, res, ctx)
        ctx.next_norm = self.norm2  # who reads the stream after the mixer has written it
        res.pending = self.mixer.forward(x, ctx, cache)
        x = self._norm(self.norm2, self.feed_forward, res, ctx)
        ctx.next_norm = getattr(ctx, "norm_after_block", None)
        res.pending = self.feed_forward.forward(x, ctx)
        ctx.residual = ctx.next_norm = None
        return res

    @staticmethod
    def _norm(norm, consumer, res: Residual, ctx):
        if norm.can_defer and consumer.wants_lazy_norm(ctx):
            return norm.forward(res, ctx, lazy=True)
        return norm.forward(res, ctx)


register_part("block", "pre_norm", PreNormBlock)
