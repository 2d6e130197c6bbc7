"""RMSNorm: y = (w * x) / sqrt(mean(x^2) + eps), statistics in float32, weight used as it is
(no 1 + w), no bias: the reference's rmsnorm_f32 (src/kernels.cpp:18-24)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .base import Norm, NormalizedRows, Residual
from .registry import register_part
from .spec import NormSpec, TensorNeed


class RMSNorm(Norm):
    def __init__(self, spec: NormSpec, env):
        super().__init__(spec, env)
        self.weight: Optional[torch.Tensor] = None

    @staticmethod
    def tensor_needs(spec: NormSpec) -> List[TensorNeed]:
        return [TensorNeed(spec.weight, (spec.dim,), "float32", init="around_one")]

    def load(self, tensors) -> None:
        self.weight = tensors[self.spec.weight]

    can_defer = True

    def forward(self, res: Residual, ctx, rows=None, n_rows=None, lazy: bool = False):
        n = ctx.n_tokens if rows is None else (rows.numel() if n_rows is None else n_rows)
        if lazy and res.pending is None and res.sumsq is not None:
            # the stream is up to date and the sums of squares of its rows are known: whoever
            # consumes the rows computes (w * x) / rms(x) while it loads them
            pre = res.prescaled if res.prescaled_weight is self.weight else None
            return NormalizedRows(res.h, res.sumsq, self.weight, self.spec.eps, rows, n, self, pre)
        out = ctx.ws.get("norm.out" if rows is None else "norm.rows_out", (n, self.spec.dim), self.env.dtype)
        self.env.ops.rmsnorm(res.h, self.weight, self.spec.eps, out, delta=res.pending, rows=rows, n_rows=n)
        if rows is None:
            if res.pending is not None:
                res.sumsq = res.prescaled = res.prescaled_weight = None  # the stream has moved on
            res.pending = None
        return out

    def prescale_weight(self):
        return self.weight

    def run(self, h: torch.Tensor, ctx, rows, n: int) -> torch.Tensor:
        """The norm's kernel on rows of a stream that has nothing pending (NormalizedRows.dense)."""
        out = ctx.ws.get("norm.out" if rows is None else "norm.rows_out", (n, self.spec.dim), self.env.dtype)
        self.env.ops.rmsnorm(h, self.weight, self.spec.eps, out, rows=rows, n_rows=n)
        return out


register_part("norm", "rmsnorm", RMSNorm)
