"""Dense gated feed-forward: down( silu(gate(x)) * up(x) ), no bias (src/engine.cpp:383-412;
silu as v/(1+exp(-v)), src/kernels.cpp:26-31). gate and up run as one product against their rows
put together: [Wg; Wu], or, in bfloat16 when the intermediate size is a multiple of 128, blocks of
128 gate rows followed by the 128 matching up rows, so that one 256-wide accumulator tile of the
tensor-core product holds both and the activation is applied in its epilogue."""
from __future__ import annotations

from typing import List, Optional

import torch

from .attention import add_into_stream_or_partials, res_sumsq_off
from .base import FeedForward, NormalizedRows
from .registry import register_part
from .spec import GatedMLPSpec, TensorNeed


class GatedMLP(FeedForward):
    def __init__(self, spec: GatedMLPSpec, env):
        super().__init__(spec, env)
        if spec.activation != "silu":
            raise ValueError(f"gated feed-forward: activation '{spec.activation}' is not implemented (silu is)")
        self.w_gate_up = None
        self.w_down = None

    @staticmethod
    def tensor_needs(spec: GatedMLPSpec) -> List[TensorNeed]:
        return [TensorNeed(spec.gate_weight, (spec.intermediate, spec.hidden)),
                TensorNeed(spec.up_weight, (spec.intermediate, spec.hidden)),
                TensorNeed(spec.down_weight, (spec.hidden, spec.intermediate))]

    def kernel_notes(self):
        s, notes = self.spec, []
        if self.env.dtype == torch.bfloat16:
            for name, k in (("gate|up", s.hidden), ("down", s.intermediate)):
                if k % 8:
                    notes.append(f"feed-forward: the {name} product sums over {k} inputs, no multiple of 8: it runs on CUDA cores")
            if s.intermediate % 128:
                notes.append(f"feed-forward: an intermediate size of {s.intermediate} is no multiple of 128: the activation is a "
                             "kernel of its own instead of the gate|up product's epilogue")
        return notes

    def load(self, tensors) -> None:
        s = self.spec
        g, u = tensors[s.gate_weight], tensors[s.up_weight]
        self.blocked = g.dtype == torch.bfloat16 and s.intermediate % 128 == 0
        if self.blocked:
            self.w_gate_up = torch.stack([g.view(-1, 128, s.hidden), u.view(-1, 128, s.hidden)], dim=1).reshape(2 * s.intermediate, s.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[s.down_weight]

    def _few_tokens(self, ctx) -> bool:
        s, ops, n = self.spec, self.env.ops, ctx.n_tokens
        return (self.blocked and hasattr(ops, "gemm_few_tokens") and
                ops.few_token_splits(2 * s.intermediate, s.hidden, n, "swiglu") > 0 and
                ops.few_token_splits(s.hidden, s.intermediate, n, "residual") > 0)

    def _takes_prescaled(self, ctx) -> bool:
        ops = self.env.ops
        return self.env.dtype == torch.bfloat16 and getattr(ops, "meet_products", False) and ctx.n_tokens <= 64

    def wants_lazy_norm(self, ctx) -> bool:
        return self._few_tokens(ctx) or self._takes_prescaled(ctx)

    def forward(self, x, ctx) -> Optional[torch.Tensor]:
        s, ops, n = self.spec, self.env.ops, ctx.n_tokens
        act = ctx.ws.get("mlp.act", (n, s.intermediate), self.env.dtype)
        if self._few_tokens(ctx):
            # few tokens: the norm before (if it was handed on), the sum of the K pieces and SiLU * up all
            # happen inside the gate|up product; the down product adds itself into the residual stream
            if isinstance(x, NormalizedRows):
                ops.gemm_few_tokens(self.w_gate_up, act, "swiglu", norm=(x.h, x.sumsq, x.weight, x.eps, x.rows), n_tokens=n, ws=ctx.ws)
            else:
                ops.gemm_few_tokens(self.w_gate_up, act, "swiglu", x=x[:n], ws=ctx.ws)
            return add_into_stream_or_partials(ops, act, self.w_down, ctx, True, "mlp.delta")
        extra = {}
        if isinstance(x, NormalizedRows):
            if (x.prescaled is not None and x.rows is None and self._takes_prescaled(ctx) and
                    ops.can_meet(x.prescaled[:n], self.w_gate_up)):
                # the product runs on weight * rows; the norm's 1/rms goes in where its partial sums are added
                extra, x = {"row_scale": x.row_scale(ops)}, x.prescaled
            else:
                x = x.dense(ctx)
        if self.blocked:
            ops.gemm_swiglu(x[:n], self.w_gate_up, act, ctx.ws, **extra)
        elif n <= 64:  # few tokens: the products may come as partial sums, added by their consumers
            ops.silu_mul_partials(ops.gemm_partials(x[:n], self.w_gate_up, ctx.ws, "mlp.gate_up_parts"), act, **extra)
        else:
            gate_up = ctx.ws.get("mlp.gate_up", (n, 2 * s.intermediate), self.env.dtype)
            ops.gemm(x[:n], self.w_gate_up, gate_up)
            ops.silu_mul(gate_up, act)
        return add_into_stream_or_partials(ops, act, self.w_down, ctx, False, "mlp.delta")


register_part("feed_forward", "gated_mlp", GatedMLP)
