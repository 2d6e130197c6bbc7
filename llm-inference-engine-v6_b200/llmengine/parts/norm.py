"""RMSNorm: y = (w * x) / sqrt(mean(x^2) + eps), statistics in float32, weight used as it is
(no 1 + w), no bias: the reference's rmsnorm_f32 (src/kernels.cpp:18-24)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .base import Norm, Residual
from .registry import register_part
from .spec import NormSpec, TensorNeed


class RMSNorm(Norm):
    def __init__(self, spec: NormSpec, env):
        super().__init__(spec, env)
        self.weight: Optional[torch.Tensor] = None

    @staticmethod
    def tensor_needs(spec: NormSpec) -> List[TensorNeed]:
        return [TensorNeed(spec.weight, (spec.dim,), "float32")]

    def load(self, tensors) -> None:
        self.weight = tensors[self.spec.weight]

    def forward(self, res: Residual, ctx, rows=None, n_rows=None) -> torch.Tensor:
        n = ctx.n_tokens if rows is None else (rows.numel() if n_rows is None else n_rows)
        out = ctx.ws.get("norm.out" if rows is None else "norm.rows_out", (n, self.spec.dim), self.env.dtype)
        self.env.ops.rmsnorm(res.h, self.weight, self.spec.eps, out, delta=res.pending, rows=rows, n_rows=n)
        if rows is None:
            res.pending = None
        return out


register_part("norm", "rmsnorm", RMSNorm)
