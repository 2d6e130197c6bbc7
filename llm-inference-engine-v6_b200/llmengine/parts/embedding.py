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

    def forward(self, x, ctx) -> torch.Tensor:
        n = x.n if isinstance(x, NormalizedRows) else x.shape[0]
        logits = ctx.ws.get("model.logits", (max(n, 1), self.spec.vocab_size), torch.float32)[:n]
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        if n:
            self.env.ops.gemm(x, self.weight, logits)
        return logits


register_part("embedding", "lookup", TokenLookup)
register_part("head", "linear", LinearHead)
