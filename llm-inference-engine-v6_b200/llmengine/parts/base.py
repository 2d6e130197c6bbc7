"""Interfaces of the parts a layer is put together from, and the objects they are handed.

No part knows which model it is in: it sees its own spec (sizes and constants), the build
environment (device, dtype, kernels), the tensors it asked for by name, and at each step the step
context (the flat batch) and, for mixers, its own layer's cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .spec import TensorNeed


@dataclass
class BuildEnv:
    device: torch.device
    dtype: torch.dtype  # engine precision: torch.float32 (true 32-bit path) or torch.bfloat16
    ops: object         # the kernel interface (llmengine.ops.CudaOps)
    page_size: int


# ---------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class KVNeed:
    """Keys and values per token, kept in pages. window 0: all of them; W: the last W.
    portion_multiple: see StateNeed."""
    num_kv_heads: int
    head_dim: int
    window: int = 0
    portion_multiple: int = 1


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, kept in the request's slot; zeroed when a request starts.
    portion_multiple: where a prompt may be cut. 1: anywhere (attention, and any state that is
    updated token by token). M > 1: a portion that leaves part of the prompt for a later step must
    end at a position that is a multiple of M (a mixer that carries its state over only at the
    edges of chunks of M tokens); the scheduler cuts prompts accordingly, and the multiple of a
    model is the least common multiple over its layers. Single decoded tokens are not portions."""
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
    portion_multiple: int = 1


@dataclass
class LayerCache:
    """What one run of a layer owns (or borrows) of the cache.
    k, v: [pages + 1, kv_heads, page_size, head_dim]; the last page is the null page that padded
    batch rows point at. group: which block table applies. writes: False when this run reads
    another run's cache. states: name -> [slots + 1, *shape]; the last slot is the null slot."""
    group: int = -1
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    writes: bool = True
    window: int = 0
    states: Dict[str, torch.Tensor] = field(default_factory=dict)


class Residual:
    """The float32 residual stream h [tokens, hidden] and a float32 delta that has not been added
    yet ([tokens, hidden], or [parts, tokens, hidden] to be summed in index order). The next norm
    adds it while it reads h, which saves one pass over the stream.

    A part whose last product can add into the stream itself (ctx.residual is the stream it works
    for) returns None instead of a delta and may leave `sumsq`: float32 [tokens, parts], the parts
    of every row's sum of squares as the stream stands now. With them a norm need not run as a
    kernel of its own: it hands NormalizedRows to a consumer that folds it into its first product."""

    def __init__(self, h: torch.Tensor):
        self.h = h
        self.pending: Optional[torch.Tensor] = None
        self.sumsq: Optional[torch.Tensor] = None  # valid only while pending is None and h is untouched since
        # beside sumsq, what the product that last added into the stream may also leave for the norm that
        # comes next (ctx.next_norm): the stream's rows times that norm's weight, in the engine dtype. The
        # norm's 1/rms is a scalar per row, so the product behind the norm can run on these rows as they
        # are and the scalar be multiplied in where that product's results are consumed (ops.RowScale).
        self.prescaled: Optional[torch.Tensor] = None
        self.prescaled_weight: Optional[torch.Tensor] = None  # the weight tensor prescaled was made with


@dataclass
class NormalizedRows:
    """What a norm hands on without having run: rows of the float32 stream, the parts of their sums
    of squares, its weight and eps; `rows` (int32) picks rows, `n` is how many. A consumer that
    takes it (wants_lazy_norm) computes (weight * x) / rms(x) itself; dense() runs the norm's kernel."""
    h: torch.Tensor
    sumsq: torch.Tensor
    weight: torch.Tensor
    eps: float
    rows: Optional[torch.Tensor]
    n: int
    norm: "Norm"
    prescaled: Optional[torch.Tensor] = None  # weight * h in the engine dtype (all rows of h), if the producer left it

    def dense(self, ctx) -> torch.Tensor:
        return self.norm.run(self.h, ctx, self.rows, self.n)

    def row_scale(self, ops):
        """The 1/rms of the rows as the kernels take it (for consumers of a product of `prescaled`)."""
        return ops.row_scale(self.sumsq, self.h.shape[1], self.eps)


class Part:
    category = ""
    # False for a part whose forward waits for the device or sizes its work from device data (a
    # .tolist(), a .nonzero()): such a step cannot be recorded as a CUDA graph, and the engine then
    # runs the model's decode steps kernel by kernel. Parts made of kernels on fixed shapes leave it True.
    capturable = True

    def __init__(self, spec, env: BuildEnv):
        self.spec = spec
        self.env = env

    def subparts(self) -> Sequence["Part"]:
        """The parts this one is made of (a block's norms, mixer and feed-forward; a mixer's position
        encoding), so that questions asked of a model reach every part."""
        return ()

    def wants_lazy_norm(self, ctx) -> bool:
        """True if, in this step, the part takes NormalizedRows in place of normalised activations."""
        return False

    def kernel_notes(self) -> List[str]:
        """One line for each thing a user should know about how this part will run at the engine's
        precision, e.g. that its sizes leave the tensor-core kernels out; shown once when the
        model is loaded."""
        return []

    @staticmethod
    def tensor_needs(spec) -> List[TensorNeed]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receives every tensor it asked for, on the device, in the asked precision."""


class Embedding(Part):
    category = "embedding"

    def forward(self, ctx) -> torch.Tensor:
        """The float32 residual stream [tokens, hidden] of the step's tokens (ctx.token_ids). It may
        leave ctx.stream_sumsq: float32 [tokens, parts], the parts of every row's sum of squares
        (see Residual.sumsq)."""
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x: the wanted rows after the final norm [rows, hidden] (engine dtype). Returns float32
        logits [rows, vocab]."""
        raise NotImplementedError


class Norm(Part):
    category = "norm"
    can_defer = False  # True: forward(..., lazy=True) may return NormalizedRows

    def prescale_weight(self) -> Optional[torch.Tensor]:
        """For a norm of the form (weight * x) * s(x) with s a scalar per row that only needs the row's
        sum of squares: the float32 weight [dim], so that whoever writes the stream last can leave
        weight * x beside it (Residual.prescaled). None (the default): this norm runs as it is."""
        return None

    def forward(self, res: Residual, ctx, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
        """Adds res.pending into res.h (when `rows` is None) and returns the normalised rows in the
        engine dtype. With `rows`, only those source rows are normalised and res is left alone.
        Norms with can_defer take `lazy=True` as well (asked for only when the consumer wants it)."""
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"

    # True if rotate_and_store takes `parts`: float32 [p, tokens, width] partial sums of the q|k|v
    # product to be added (in index order) while encoding, instead of finished values in qkv.
    takes_partial_sums = False
    # True if rotate_and_store also takes `row_scale` beside `parts` (when the layer writes its cache):
    # a scalar per token that the sums are multiplied with before anything else (ops.RowScale).
    takes_row_scale = False

    def rotation_tables(self):
        """For mixers that fold the encoding into their own kernel: (cos, sin) float32 tables
        [positions, head_dim / 2] of a half-split rotation, (None, None) if nothing is rotated, or
        None (the default) if the encoding is not of that form and rotate_and_store must be used."""
        return None

    def rotate_and_store(self, qkv: torch.Tensor, ctx, cache: LayerCache, num_heads: int, num_kv_heads: int,
                         head_dim: int, parts: Optional[torch.Tensor] = None) -> None:
        """Encodes positions into q and k of qkv [tokens, (heads + 2 kv_heads) * head_dim] in place
        and writes k, v of every token into its page of `cache` (if cache.writes)."""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    def cache_needs(self) -> Sequence[object]:
        """KVNeed / StateNeed objects; empty if the mixer keeps nothing between steps."""
        return ()

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache) -> torch.Tensor:
        """x: normalised activations [tokens, hidden] (engine dtype). Returns the float32 delta to
        be added to the residual stream: [tokens, hidden], or [parts, tokens, hidden] partial sums."""
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """As Mixer.forward, without a cache."""
        raise NotImplementedError


class Block(Part):
    category = "block"

    def cache_needs(self) -> Sequence[object]:
        return ()

    def first_norm(self) -> Optional[Norm]:
        """The norm that reads the residual stream first in this block, if the block begins with one: the
        model tells the part that writes the stream before it (ctx.next_norm)."""
        return None

    def forward(self, res: Residual, ctx, cache: LayerCache) -> Residual:
        """ctx.norm_after_block: the norm that reads the stream after this block (the next block's
        first, or the model's final norm), or None."""
        raise NotImplementedError
