"""Position encodings.

"rope": rotary encoding in the half-split layout with optional Llama-3 frequency rescaling. The
tables are built on the host exactly as the reference builds them: inverse frequencies in float64
rounded to float32 (llama3_inv_freq, src/kernels.cpp:114-160, with pi taken as the float constant),
angle = double(p) * double(inv_freq_f32), cos/sin in float64 rounded to float32
(build_rope_tables, src/kernels.cpp:162-187). The table has one row per position up to the
model's position limit; the reference's cap at 8192 rows is not kept.
"none": stores k and v unrotated.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import LayerCache, PositionEncoding
from .registry import register_part
from .spec import PositionSpec

_PI_F32 = float(np.float32(3.14159265358979323846))


def rope_inverse_frequencies(spec: PositionSpec) -> np.ndarray:
    half = spec.head_dim // 2
    theta = float(spec.theta)
    inv = [1.0 / math.pow(theta, (2 * i) / spec.head_dim) for i in range(half)]
    if spec.original_max_positions > 0:
        orig = float(spec.original_max_positions)
        factor, low_f, high_f = float(spec.scaling_factor), float(spec.low_freq_factor), float(spec.high_freq_factor)
        low_wavelen, high_wavelen = orig / low_f, orig / high_f
        for i, fr in enumerate(inv):
            wavelen = 2.0 * _PI_F32 / fr
            if wavelen > low_wavelen:
                inv[i] = fr / factor
            elif wavelen >= high_wavelen:
                smooth = (orig / wavelen - low_f) / (high_f - low_f)
                inv[i] = (1.0 - smooth) * fr / factor + smooth * fr
    return np.asarray(inv, dtype=np.float64).astype(np.float32)


def rope_tables(spec: PositionSpec):
    """-> cos, sin as float32 arrays [max_positions, head_dim / 2]."""
    inv = rope_inverse_frequencies(spec).astype(np.float64)
    ang = np.arange(spec.max_positions, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


# One pair of tables per (spec, device), whichever and however many layers use it: the layers of a
# model share one position spec, and a table of 131,072 positions with head size 128 is 67 MB.
_TABLES = {}


def shared_rope_tables(spec: PositionSpec, device: torch.device):
    key = (spec, str(device))
    hit = _TABLES.get(key)
    if hit is None:
        cos, sin = rope_tables(spec)
        hit = (torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device))
        while len(_TABLES) >= 8:  # engines come and go in one process (tests): the oldest entries go
            _TABLES.pop(next(iter(_TABLES)))
        _TABLES[key] = hit
    return hit


class RotaryPosition(PositionEncoding):
    takes_partial_sums = True

    def __init__(self, spec: PositionSpec, env):
        super().__init__(spec, env)
        if spec.head_dim <= 0 or spec.head_dim % 2:
            raise ValueError(f"rotary position encoding needs an even head_dim, got {spec.head_dim}")
        if spec.max_positions <= 0:
            raise ValueError("rotary position encoding needs max_positions >= 1")
        self.cos, self.sin = shared_rope_tables(spec, env.device)

    def rotation_tables(self):
        return self.cos, self.sin

    takes_row_scale = True

    def rotate_and_store(self, qkv, ctx, cache: LayerCache, num_heads, num_kv_heads, head_dim, parts=None, row_scale=None) -> None:
        write = cache.writes and cache.k is not None
        extra = {} if row_scale is None else {"row_scale": row_scale}
        self.env.ops.rope_kv_write(qkv, ctx.positions, ctx.token_seq, ctx.block_tables[cache.group], self.cos, self.sin,
                                   cache.k if write else None, cache.v if write else None, ctx.n_tokens, num_heads,
                                   num_kv_heads, head_dim, parts=parts, **extra)


class NoPosition(PositionEncoding):
    takes_partial_sums = True

    def rotation_tables(self):
        return None, None

    takes_row_scale = True

    def rotate_and_store(self, qkv, ctx, cache: LayerCache, num_heads, num_kv_heads, head_dim, parts=None, row_scale=None) -> None:
        if cache.writes and cache.k is not None:
            extra = {} if row_scale is None else {"row_scale": row_scale}
            self.env.ops.rope_kv_write(qkv, ctx.positions, ctx.token_seq, ctx.block_tables[cache.group], None, None,
                                       cache.k, cache.v, ctx.n_tokens, num_heads, num_kv_heads, head_dim, parts=parts, **extra)
        elif parts is not None:
            assert row_scale is None, "a row scale is taken only where the layer writes its cache"
            self.env.ops.reduce_partials(parts, qkv)


register_part("position", "rope", RotaryPosition)
register_part("position", "none", NoPosition)
