"""Choosing the next token from logits rows, on the device.

Greedy: first index of the maximum (the reference's only sampler, src/engine.cpp:52-58).
Temperature T > 0: a draw from softmax(logits / T) taken as argmax(logits / T + Gumbel noise),
the noise a pure function of (request seed, index of the draw within the request, token index);
so the same request yields the same tokens whatever else is batched with it. T = 0 is greedy.
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch


class Sampler:
    def __init__(self, ops, device: torch.device):
        self.wait_seconds = 0.0  # host time spent waiting for the device to finish a step (statistics)
        self.ops, self.device = ops, device
        self._out: Optional[torch.Tensor] = None
        self._host: Optional[torch.Tensor] = None
        self._scratch: Optional[torch.Tensor] = None

    def _buffers(self, n: int):
        if self._out is None or self._out.numel() < n:
            cap = max(64, 1 << (n - 1).bit_length())
            self._out = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._host = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        return self._out, self._host

    def _scratch_for(self, n: int, vocab: int):
        if not hasattr(self.ops, "sample_scratch_words"):
            return None
        words = self.ops.sample_scratch_words(n, vocab)
        if self._scratch is None or self._scratch.numel() < words:
            self._scratch = torch.empty(max(words, 1024), dtype=torch.int32, device=self.device)
        return self._scratch

    def sample_device(self, logits: torch.Tensor, ctx, n_rows: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """-> int32 tensor [rows]; the rows' parameters come from the step's batch. `out` may be given:
        a device tensor, or pinned host memory that the kernel writes through its mapped address (the
        host then needs no copy, only to wait for the stream)."""
        n = logits.shape[0] if n_rows is None else n_rows
        if out is None:
            out, _ = self._buffers(max(n, 1))
        if n:
            self.ops.sample(logits, out, ctx.row_temperature, ctx.row_seed, ctx.row_draw, n_rows=n,
                            scratch=self._scratch_for(n, logits.shape[1]))
        return out[:n]

    def sample(self, logits: torch.Tensor, ctx, n_rows: Optional[int] = None) -> List[int]:
        """-> token ids on the host (one device-to-host copy of 4 bytes a row)."""
        n = logits.shape[0] if n_rows is None else n_rows
        if n == 0:
            return []
        dev = self.sample_device(logits, ctx, n)
        _, host = self._buffers(n)
        host[:n].copy_(dev, non_blocking=True)
        if self.device.type == "cuda":
            t0 = time.perf_counter()
            torch.cuda.current_stream().synchronize()
            self.wait_seconds += time.perf_counter() - t0
        return host[:n].tolist()

    def greedy(self, logits: torch.Tensor) -> List[int]:
        n = logits.shape[0]
        if n == 0:
            return []
        out, _ = self._buffers(n)
        self.ops.sample(logits, out, None, None, None, n_rows=n, scratch=self._scratch_for(n, logits.shape[1]))
        return out[:n].tolist()
