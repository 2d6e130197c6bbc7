"""Causal grouped-query attention over the paged cache.

q, k, v projections without bias (src/engine.cpp:319-341) as one product against the row-wise
concatenation [Wq; Wk; Wv] (each output element is the same dot as with three products), position
encoding on q and k, k (encoded) and v written to the cache (src/engine.cpp:343-353), attention of
every token over cache positions lo..pos of its request (src/kernels.cpp:413-474), output
projection (src/engine.cpp:364-379). The residual sum is left to the caller.
"""
from __future__ import annotations

import math
from typing import List

import torch

from .base import KVNeed, LayerCache, Mixer
from .registry import build_part, part_class, register_part
from .spec import AttentionSpec, TensorNeed


class PagedAttention(Mixer):
    def __init__(self, spec: AttentionSpec, env):
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"attention: {spec.num_heads} heads cannot share {spec.num_kv_heads} key/value heads")
        if spec.window < 0:
            raise ValueError("attention: window must be >= 0")
        self.position = build_part("position", spec.position, env)
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)
        self.w_qkv = None
        self.w_o = None

    @staticmethod
    def tensor_needs(spec: AttentionSpec) -> List[TensorNeed]:
        dq, dkv = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        return [TensorNeed(spec.q_weight, (dq, spec.hidden)), TensorNeed(spec.k_weight, (dkv, spec.hidden)),
                TensorNeed(spec.v_weight, (dkv, spec.hidden)), TensorNeed(spec.o_weight, (spec.hidden, dq))] + \
            list(part_class("position", spec.position.kind).tensor_needs(spec.position))

    def cache_needs(self):
        return (KVNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window),)

    def load(self, tensors) -> None:
        s = self.spec
        self.w_qkv = torch.cat([tensors[s.q_weight], tensors[s.k_weight], tensors[s.v_weight]], dim=0).contiguous()
        self.w_o = tensors[s.o_weight]
        self.position.load(tensors)

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache) -> torch.Tensor:
        s, ops, n = self.spec, self.env.ops, ctx.n_tokens
        dq, dkv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        qkv = ctx.ws.get("attention.qkv", (n, dq + 2 * dkv), self.env.dtype)
        att = ctx.ws.get("attention.out", (n, dq), self.env.dtype)
        if n <= 64 and cache.writes and self.position.takes_partial_sums:
            # few tokens: the product comes as K-split partial sums, added by the position kernel
            parts = ops.gemm_partials(x[:n], self.w_qkv, ctx.ws, "attention.qkv_parts")
            tables = self.position.rotation_tables() if cache.k is not None else None
            if tables is not None and ops.decode_attention_fusable(ctx, cache.k, s.num_heads, s.num_kv_heads, s.head_dim, att):
                # single decoded tokens: summing the parts, rotation and the cache write happen inside the attention kernel
                ops.paged_attention_decode_fused(parts, tables[0], tables[1], cache.k, cache.v, ctx,
                                                 ctx.block_tables[cache.group], att, s.num_heads, s.num_kv_heads,
                                                 s.head_dim, self.scale, s.window)
                return ops.gemm_partials(att, self.w_o, ctx.ws, "attention.delta")
            self.position.rotate_and_store(qkv, ctx, cache, s.num_heads, s.num_kv_heads, s.head_dim, parts=parts)
        else:
            ops.gemm(x[:n], self.w_qkv, qkv, ctx.ws)
            self.position.rotate_and_store(qkv, ctx, cache, s.num_heads, s.num_kv_heads, s.head_dim)
        ops.paged_attention(qkv[:, :dq], cache.k, cache.v, ctx, ctx.block_tables[cache.group], att, s.num_heads,
                            s.num_kv_heads, s.head_dim, self.scale, s.window)
        return ops.gemm_partials(att, self.w_o, ctx.ws, "attention.delta")


register_part("mixer", "attention", PagedAttention)
