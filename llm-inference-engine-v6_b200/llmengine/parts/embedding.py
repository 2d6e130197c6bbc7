"""Token embedding and output head.

"lookup": the residual stream starts as the table row of each token id, widened to float32
(embed_lookup_f32, src/kernels.cpp:59-66). "linear": logits = x . W^T without bias for the rows
whose logits are wanted (src/engine.cpp:415-433); with tied embeddings W is the embedding table
itself (src/model.cpp:184-195). Variants (a scaled embedding, a capped or biased head) are other
registered kinds; the model only knows the two interfaces.
"""
from __future__ import annotations

from typing import List

import torch

from .base import Embedding, Head, NormalizedRows
from .registry import register_part
from .spec import EmbeddingSpec, HeadSpec, TensorNeed


class TokenLookup(Embedding):
    def __init__(self, spec: EmbeddingSpec, env):
        super().__init__(spec, env)
        self.table = None

    @staticmethod
    def tensor_needs(spec: EmbeddingSpec) -> List[TensorNeed]:
        return [TensorNeed(spec.weight, (spec.vocab_size, spec.dim), "compute")]

    def load(self, tensors) -> None:
        self.table = tensors[self.spec.weight]

    def forward(self, ctx) -> torch.Tensor:
        ops, n = self.env.ops, ctx.n_tokens
        h = ctx.ws.get("model.residual", (n, self.spec.dim), torch.float32)
        nxt = getattr(ctx, "next_norm", None)
        wn = nxt.prescale_weight() if nxt is not None else None
        if (self.env.dtype == torch.bfloat16 and getattr(ops, "meet_products", False) and n <= 64 and wn is not None and
                wn.numel() == self.spec.dim and wn.dtype == torch.float32):
            # a step of few tokens: the gather has the rows in its hands, so it leaves what the first norm
            # needs beside them (its weight times the rows, and the rows' sums of squares), and that norm
            # is no kernel of its own
            ctx.stream_sumsq = ctx.ws.get("embedding.sumsq", (n, 1), torch.float32)
            scaled = ctx.ws.get("stream.prescaled", (n, self.spec.dim), torch.bfloat16)
            ctx.stream_prescaled = (scaled, wn)
            return ops.embed(self.table, ctx.token_ids, h, sumsq=ctx.stream_sumsq, next_w=wn, scaled=scaled)
        if self.env.dtype == torch.bfloat16 and hasattr(ops, "few_token_splits") and ops.few_token_splits(128, self.spec.dim, n, "plain") > 0:
            # a step of few tokens: the first norm can be folded into the product after it if the
            # rows' sums of squares are known; the gather has the rows in its hands anyway
            ctx.stream_sumsq = ctx.ws.get("embedding.sumsq", (n, 1), torch.float32)
            return ops.embed(self.table, ctx.token_ids, h, sumsq=ctx.stream_sumsq)
        return ops.embed(self.table, ctx.token_ids, h)


class LinearHead(Head):
    def __init__(self, spec: HeadSpec, env):
        super().__init__(spec, env)
        self.weight = None

    @staticmethod
    def tensor_needs(spec: HeadSpec) -> List[TensorNeed]:
        return [TensorNeed(spec.weight, (spec.vocab_size, spec.dim), "compute")]

    def load(self, tensors) -> None:
        self.weight = tensors[self.spec.weight]

    def wants_lazy_norm(self, ctx) -> bool:
        # every request of the step brings one token and wants its logits: the wanted rows are all rows, in order
        return (self.env.dtype == torch.bfloat16 and getattr(self.env.ops, "meet_products", False) and
                0 < ctx.n_rows == ctx.n_tokens == ctx.n_seqs <= 64)

    def forward(self, x, ctx) -> torch.Tensor:
        n = x.n if isinstance(x, NormalizedRows) else x.shape[0]
        logits = ctx.ws.get("model.logits", (max(n, 1), self.spec.vocab_size), torch.float32)[:n]
        if isinstance(x, NormalizedRows):
            ops = self.env.ops
            if x.prescaled is not None and n and self.wants_lazy_norm(ctx) and ops.can_meet(x.prescaled[:n], self.weight):
                # the product runs on weight * rows and divides by the rows' root mean square in its epilogue
                return ops.gemm_scaled(x.prescaled[:n], self.weight, logits, x.row_scale(ops))
            x = x.dense(ctx)
        if n:
            self.env.ops.gemm(x, self.weight, logits)
        return logits


register_part("embedding", "lookup", TokenLookup)
register_part("head", "linear", LinearHead)
