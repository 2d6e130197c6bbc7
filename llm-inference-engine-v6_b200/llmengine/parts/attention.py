"""Causal grouped-query attention over the paged cache.

q, k, v projections without bias (src/engine.cpp:319-341) as one product against the row-wise
concatenation [Wq; Wk; Wv] (each output element is the same dot as with three products), position
encoding on q and k, k (encoded) and v written to the cache (src/engine.cpp:343-353), attention of
every token over cache positions lo..pos of its request (src/kernels.cpp:413-474), output
projection (src/engine.cpp:364-379). The residual sum is left to the caller.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .base import KVNeed, LayerCache, Mixer, NormalizedRows
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

    def subparts(self):
        return (self.position,)

    def cache_needs(self):
        return (KVNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window),)

    def kernel_notes(self):
        s, notes = self.spec, []
        if self.env.dtype == torch.bfloat16 and hasattr(self.env.ops, "attention_kernels"):
            prompt, decode = self.env.ops.attention_kernels(s.num_heads, s.num_kv_heads, s.head_dim, self.env.page_size)
            for what, kernel in (("prompt portions", prompt), ("single decoded tokens", decode)):
                if kernel != "tensor cores":
                    notes.append(f"attention with head size {s.head_dim}, {s.num_heads // s.num_kv_heads} query heads a key/value "
                                 f"head and pages of {self.env.page_size}: {what} run on {kernel}")
            for name, k in (("q|k|v", s.hidden), ("o", s.num_heads * s.head_dim)):
                if k % 8:
                    notes.append(f"attention: the {name} product sums over {k} inputs, no multiple of 8: it runs on CUDA cores")
        return notes

    def load(self, tensors) -> None:
        s = self.spec
        self.w_qkv = torch.cat([tensors[s.q_weight], tensors[s.k_weight], tensors[s.v_weight]], dim=0).contiguous()
        self.w_o = tensors[s.o_weight]
        self.position.load(tensors)

    def _few_tokens(self, ctx) -> bool:
        """The step has few enough tokens for the products that add their K pieces inside a cluster and
        take the work around them in (ops.gemm_few_tokens)."""
        s, ops, n = self.spec, self.env.ops, ctx.n_tokens
        return (self.env.dtype == torch.bfloat16 and hasattr(ops, "gemm_few_tokens") and
                ops.few_token_splits(self.w_qkv.shape[0], s.hidden, n, "plain") > 0 and
                ops.few_token_splits(s.hidden, s.num_heads * s.head_dim, n, "residual") > 0)

    def _takes_prescaled(self, ctx) -> bool:
        """The step has few enough tokens for the q|k|v product to come as partial sums, and whoever
        finishes them (the attention kernel or the position encoding) takes the norm's 1/rms as a row scale."""
        ops = self.env.ops
        return (self.env.dtype == torch.bfloat16 and getattr(ops, "meet_products", False) and ctx.n_tokens <= 64 and
                self.position.takes_partial_sums and self.position.takes_row_scale)

    def wants_lazy_norm(self, ctx) -> bool:
        return (self._few_tokens(ctx) and self.position.takes_partial_sums) or self._takes_prescaled(ctx)

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n = self.spec, self.env.ops, ctx.n_tokens
        dq, dkv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        qkv = ctx.ws.get("attention.qkv", (n, dq + 2 * dkv), self.env.dtype)
        att = ctx.ws.get("attention.out", (n, dq), self.env.dtype)
        few = self._few_tokens(ctx)
        row_scale = None
        if isinstance(x, NormalizedRows):
            if (x.prescaled is not None and x.rows is None and cache.writes and cache.k is not None and self._takes_prescaled(ctx)
                    and ops.can_meet(x.prescaled[:n], self.w_qkv)):
                # the rows times the norm's weight are there already: the product runs on them, and the
                # norm's 1/rms goes in where the product's partial sums are finished
                row_scale, x, few = x.row_scale(ops), x.prescaled, False
            elif not (few and cache.writes and self.position.takes_partial_sums):
                x = x.dense(ctx)
        if n <= 64 and cache.writes and self.position.takes_partial_sums:
            # few tokens: the product comes as float32 sums (in parts, unless the K pieces were added
            # inside the product), finished by the position kernel or by the attention kernel
            if few:
                parts = ctx.ws.get("attention.qkv_parts", (1, n, dq + 2 * dkv), torch.float32)
                if isinstance(x, NormalizedRows):
                    ops.gemm_few_tokens(self.w_qkv, parts[0], "plain", norm=(x.h, x.sumsq, x.weight, x.eps, x.rows), n_tokens=n, ws=ctx.ws)
                else:
                    ops.gemm_few_tokens(self.w_qkv, parts[0], "plain", x=x[:n], ws=ctx.ws)
            else:
                parts = ops.gemm_partials(x[:n], self.w_qkv, ctx.ws, "attention.qkv_parts")
            tables = self.position.rotation_tables() if cache.k is not None else None
            if tables is not None and ops.decode_attention_fusable(ctx, cache.k, s.num_heads, s.num_kv_heads, s.head_dim, att):
                # single decoded tokens: summing the parts, rotation and the cache write happen inside the attention kernel
                extra = {} if row_scale is None else {"row_scale": row_scale}
                ops.paged_attention_decode_fused(parts, tables[0], tables[1], cache.k, cache.v, ctx,
                                                 ctx.block_tables[cache.group], att, s.num_heads, s.num_kv_heads,
                                                 s.head_dim, self.scale, s.window, **extra)
                return self._output(att, ctx, few)
            extra = {} if row_scale is None else {"row_scale": row_scale}
            self.position.rotate_and_store(qkv, ctx, cache, s.num_heads, s.num_kv_heads, s.head_dim, parts=parts, **extra)
        else:
            ops.gemm(x[:n], self.w_qkv, qkv, ctx.ws)
            self.position.rotate_and_store(qkv, ctx, cache, s.num_heads, s.num_kv_heads, s.head_dim)
        ops.paged_attention(qkv[:, :dq], cache.k, cache.v, ctx, ctx.block_tables[cache.group], att, s.num_heads,
                            s.num_kv_heads, s.head_dim, self.scale, s.window)
        return self._output(att, ctx, few)

    def _output(self, att: torch.Tensor, ctx, few: bool) -> Optional[torch.Tensor]:
        """The output projection: added into the residual stream by the product itself where that
        applies (returns None), else float32 partial sums for the next norm to add."""
        return add_into_stream_or_partials(self.env.ops, att, self.w_o, ctx, few, "attention.delta")


def add_into_stream_or_partials(ops, x: torch.Tensor, w: torch.Tensor, ctx, few: bool, tag: str) -> Optional[torch.Tensor]:
    """A sub-layer's last product x . w^T. With few tokens, and a residual stream to work for, the
    product adds itself into the stream and leaves the parts of the rows' sums of squares there
    (so that the next norm need not run); otherwise it returns float32 partial sums."""
    res, n = ctx.residual, ctx.n_tokens
    if (not few and res is not None and res.pending is None and res.h.shape[1] == w.shape[0] and x.dtype == torch.bfloat16 and
            hasattr(ops, "gemm_meet") and ops.can_meet(x[:n], w)):
        # few tokens: the K splits meet inside the product, which adds their sum into the stream and
        # leaves, for the norm that reads the stream next, its weight times the stream and the parts of
        # the rows' sums of squares
        nxt = getattr(ctx, "next_norm", None)
        wn = nxt.prescale_weight() if nxt is not None else None
        if wn is not None and (wn.numel() != w.shape[0] or wn.dtype != torch.float32):
            wn = None
        ss = ctx.ws.get("stream.sumsq", (res.h.shape[0], (w.shape[0] + 127) // 128), torch.float32)
        scaled = ctx.ws.get("stream.prescaled", tuple(res.h.shape), torch.bfloat16) if wn is not None else None
        ops.gemm_meet(x[:n], w, res.h, ctx.ws, tag, next_w=wn, scaled=scaled, sumsq=ss)
        res.sumsq, res.prescaled, res.prescaled_weight = ss, scaled, wn
        return None
    if (not few and res is not None and res.pending is None and res.h.shape[1] == w.shape[0] and x.dtype == torch.bfloat16 and
            hasattr(ops, "gemm_add_into") and ops.can_add_into(x[:n], w)):
        # a prompt-sized step: the product's epilogue adds into the stream (the same float32 sums as the
        # next norm would have made from the product written out)
        res_sumsq_off(res)
        ops.gemm_add_into(x[:n], w, res.h)
        return None
    if few and res is not None and res.pending is None and res.h.shape[1] == w.shape[0]:
        parts = ops.residual_sumsq_parts(w.shape[0], w.shape[1], n)
        ss = ctx.ws.get(tag + ".sumsq", (res.h.shape[0], parts), torch.float32)
        ops.gemm_few_tokens(w, res.h, "residual", x=x[:n], sumsq_out=ss, n_tokens=n, ws=ctx.ws)
        res.sumsq, res.prescaled, res.prescaled_weight = ss, None, None
        return None
    res_sumsq_off(res)
    return ops.gemm_partials(x, w, ctx.ws, tag)


def res_sumsq_off(res) -> None:
    if res is not None:  # a delta is on its way: what was left beside the stream no longer describes it
        res.sumsq = res.prescaled = res.prescaled_weight = None


register_part("mixer", "attention", PagedAttention)
