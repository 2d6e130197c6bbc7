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
        h = ctx.ws.get("model.residual", (ctx.n_tokens, self.spec.dim), torch.float32)
        return self.env.ops.embed(self.table, ctx.token_ids, h)


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
        ops = self.env.ops
        return (self.env.dtype == torch.bfloat16 and hasattr(ops, "gemm_few_tokens") and
                ops.few_token_splits(self.spec.vocab_size, self.spec.dim, ctx.n_rows, "plain") > 0)

    def forward(self, x, ctx) -> torch.Tensor:
        n = x.n if isinstance(x, NormalizedRows) else x.shape[0]
        logits = ctx.ws.get("model.logits", (max(n, 1), self.spec.vocab_size), torch.float32)[:n]
        if isinstance(x, NormalizedRows):  # the final norm of the wanted rows happens inside the product
            self.env.ops.gemm_few_tokens(self.weight, logits, "plain", norm=(x.h, x.sumsq, x.weight, x.eps, x.rows), n_tokens=n)
        elif n:
            self.env.ops.gemm(x, self.weight, logits)
        return logits


register_part("embedding", "lookup", TokenLookup)
register_part("head", "linear", LinearHead)
