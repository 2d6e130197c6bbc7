"""What a step hands to the parts: the flat batch on the device, and scratch memory.

The batch is one int32 buffer, filled on the host by the C++ batch builder into pinned memory and
copied to the device in one transfer; the arrays below are views into the device copy.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.host import host_module


class Workspace:
    """Scratch tensors by tag. A tag's buffer grows to the largest size asked for and is then
    reused by every step (and every layer that uses the tag), so steady-state steps allocate
    nothing and addresses stay fixed for CUDA-graph replays."""

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[str, torch.Tensor] = {}
        self.frozen = False  # set while a CUDA graph is being captured or replayed

    def get(self, tag: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        buf = self._buffers.get(tag)
        if buf is None or buf.numel() < nbytes:
            if self.frozen:
                raise RuntimeError(f"workspace '{tag}' would have to grow while a CUDA graph depends on it")
            buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=self.device)
            self._buffers[tag] = buf
        return buf[:nbytes].view(dtype).view(shape)

    def get_zeroed(self, tag: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """As get, for memory that must read zero the first time: the buffer is cleared when it is
        made (or grown), not at every call; its users leave it zero again."""
        before = self._buffers.get(tag)
        out = self.get(tag, shape, dtype)
        if self._buffers.get(tag) is not before:
            self._buffers[tag].zero_()
        return out

    def zero(self, tag: str) -> None:
        """Clears a tag's buffer, if there is one (after a failed step left it in an unknown state)."""
        buf = self._buffers.get(tag)
        if buf is not None:
            buf.zero_()

    def bytes(self) -> int:
        return sum(b.numel() for b in self._buffers.values())


class StepContext:
    """One step's batch as the parts see it. Host-side counts are plain ints; everything else is
    an int32 device tensor.
      token_ids, positions, token_seq [n_tokens]: id, absolute position and batch row of each token
      seq_start, seq_ntok, seq_len, seq_slot [n_seqs]; seq_qoff [n_seqs+1]: per request of the batch
      block_tables[g] [n_seqs, max_blocks]: page of positions [i*page, (i+1)*page) in cache group g
      logit_rows [n_rows]: flat token rows whose logits are wanted
      row_temperature (float32 view), row_seed, row_draw [n_rows]: sampling parameters of those rows
    """

    def __init__(self):
        self.n_tokens = self.n_seqs = self.n_rows = 0
        self.max_seq_len = self.max_new_tokens = 0
        self.decode_only = False
        self.page_size = 0
        self.ws: Optional[Workspace] = None
        self.token_ids = self.positions = self.token_seq = self.logit_rows = None
        self.row_temperature = self.row_seed = self.row_draw = None
        self.seq_start = self.seq_ntok = self.seq_qoff = self.seq_slot = self.seq_len = None
        self.block_tables: List[torch.Tensor] = []
        self.stream_sumsq = None  # left by the embedding for the first norm (parts.base.Embedding.forward)
        self.residual = None  # the stream (parts.base.Residual) that the part being run works for, if it may add into it
        self.stream_prescaled = None  # (rows times the first norm's weight, that weight), left by the embedding likewise
        self.next_norm = None  # the norm that reads the stream after the part being run has written it, if known
        self.norm_after_block = None  # the norm that reads the stream after the block being run


class StepBuffers:
    """Pinned host staging and its device twin for the step's int32 arrays."""

    def __init__(self, device: torch.device, num_groups: int, page_size: int, ws: Workspace):
        self.device, self.num_groups, self.page_size, self.ws = device, num_groups, page_size, ws
        self.host: Optional[torch.Tensor] = None
        self.dev: Optional[torch.Tensor] = None
        self._copied = None  # event: the last host->device copy has finished reading `host`
        self.h2d_bytes = 0   # bytes of the last transfer (for measurements)
        self._views = None   # (elements, device view, host view) of the last refill

    def _ensure(self, total: int) -> None:
        if self.host is None or self.host.numel() < total:
            cap = max(1024, 1 << (total - 1).bit_length())
            if self._copied is not None:
                self._copied.synchronize()
            on_gpu = self.device.type == "cuda"
            self._views = None
            self.host = torch.empty(cap, dtype=torch.int32, pin_memory=on_gpu)
            self.dev = torch.empty(cap, dtype=torch.int32, device=self.device)

    def prepare(self, cm, entries, vocab_size: int, max_positions: int, pad_to: Optional[Tuple[int, int, int, int]] = None) -> StepContext:
        """Builds the batch of `entries` (pages already reserved) and starts its copy to the device.
        pad_to = (tokens, requests, rows, blocks) fixes the capacities and pads the batch to them."""
        H = host_module()
        if pad_to is None:
            tokens, seqs, rows, blocks = H.step_caps(cm, entries)
            caps = (max(tokens, 1), max(seqs, 1), max(rows, 1), blocks)
        else:
            caps = pad_to
        layout = H.StepLayout.make(caps[0], caps[1], caps[2], caps[3], self.num_groups)
        self._ensure(layout.total)
        if self._copied is not None:
            self._copied.synchronize()
        counts = H.fill_step(cm, entries, layout, self.host.data_ptr(), pad_to is not None, vocab_size, max_positions)
        self.dev[:layout.total].copy_(self.host[:layout.total], non_blocking=True)
        if self.device.type == "cuda":
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()
        self.h2d_bytes = layout.total * 4
        return self.context(layout, counts, padded=pad_to is not None)

    def refill(self, cm, entries, layout, vocab_size: int, max_positions: int):
        """The same arrays for the next step of a padded batch whose layout (and so every device
        address) stays as the last prepare() left it: a captured graph keeps reading the tensors of
        that call's context, so nothing but the fill and the copy has to happen. -> the step's counts."""
        self._copied.synchronize()
        H = host_module()
        counts = H.fill_step(cm, entries, layout, self.host.data_ptr(), True, vocab_size, max_positions)
        if self._views is None or self._views[0] != layout.total:
            self._views = (layout.total, self.dev[:layout.total], self.host[:layout.total])
        self._views[1].copy_(self._views[2], non_blocking=True)
        self._copied.record()
        self.h2d_bytes = layout.total * 4
        return counts

    def context(self, layout, counts, padded: bool) -> StepContext:
        d = self.dev
        c = StepContext()
        c.ws, c.page_size = self.ws, self.page_size
        c.n_tokens = layout.cap_tokens if padded else counts.n_tokens
        c.n_seqs = layout.cap_seqs if padded else counts.n_seqs
        c.n_rows = layout.cap_rows if padded else counts.n_rows
        c.real_rows = counts.n_rows
        c.max_seq_len, c.max_new_tokens, c.decode_only = counts.max_seq_len, counts.max_new_tokens, counts.decode_only
        nt, ns, nr = layout.cap_tokens, layout.cap_seqs, layout.cap_rows
        c.token_ids = d[layout.token_ids:layout.token_ids + nt]
        c.positions = d[layout.positions:layout.positions + nt]
        c.token_seq = d[layout.token_seq:layout.token_seq + nt]
        c.logit_rows = d[layout.logit_rows:layout.logit_rows + nr]
        c.row_temperature = d[layout.row_temperature:layout.row_temperature + nr].view(torch.float32)
        c.row_seed = d[layout.row_seed:layout.row_seed + nr]
        c.row_draw = d[layout.row_draw:layout.row_draw + nr]
        c.seq_start = d[layout.seq_start:layout.seq_start + ns]
        c.seq_ntok = d[layout.seq_ntok:layout.seq_ntok + ns]
        c.seq_qoff = d[layout.seq_qoff:layout.seq_qoff + ns + 1]
        c.seq_slot = d[layout.seq_slot:layout.seq_slot + ns]
        c.seq_len = d[layout.seq_len:layout.seq_len + ns]
        per = ns * layout.max_blocks
        c.block_tables = [d[layout.block_tables + g * per: layout.block_tables + (g + 1) * per].view(ns, layout.max_blocks)
                          for g in range(layout.num_groups)]
        return c
