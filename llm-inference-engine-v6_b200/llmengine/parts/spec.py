"""Descriptions of a model as data: which parts each layer is made of, with every size and
constant as a parameter, and the order in which layers run.

A description is built from a typed configuration by the architecture's `describe` function; no
part class is touched until the model is built. Each spec names its `kind`; the part registry
(parts/registry.py) maps (category, kind) to the class that implements it, so a new mixer,
feed-forward, norm or position encoding is a new spec class plus one registered part class, and a
model may use different kinds in different layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, FrozenSet, Optional, Tuple


@dataclass(frozen=True)
class TensorNeed:
    """One checkpoint tensor a part reads.
    precision: "compute" = a matrix that feeds matrix products, kept in the engine's dtype
               (bfloat16, or float32 on the 32-bit path);
               "float32" = always widened to float32 (norm weights and other vectors);
               "stored"  = kept as the file stores it (32-bit stays 32-bit, integer tables int32).
    init: what the random-weights mode draws for it: "normal" = N(0, std); "around_one" = N(1, std)
          (weights that multiply, such as a norm's); "zeros" (biases and other additive terms)."""
    name: str
    shape: Tuple[int, ...]
    precision: str = "compute"
    init: str = "normal"


@dataclass(frozen=True)
class NormSpec:
    kind: str
    dim: int
    eps: float
    weight: str  # checkpoint tensor name


@dataclass(frozen=True)
class PositionSpec:
    """kind "rope": rotary, half-split layout; `scaling` as in the configuration; kind "none"."""
    kind: str
    head_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    scaling_factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_positions: int = 0  # 0: no rescaling of frequencies


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention. window = 0 keeps every key; W > 0 reads the last W."""
    kind: str
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: PositionSpec
    q_weight: str
    k_weight: str
    v_weight: str
    o_weight: str
    window: int = 0
    scale: Optional[float] = None  # None: 1/sqrt(head_dim)


@dataclass(frozen=True)
class GatedMLPSpec:
    """down( act(gate(x)) * up(x) ), dense, no bias. activation "silu"."""
    kind: str
    hidden: int
    intermediate: int
    gate_weight: str
    up_weight: str
    down_weight: str
    activation: str = "silu"


@dataclass(frozen=True)
class BlockSpec:
    """kind "pre_norm": h += mixer(norm1(h)); h += feed_forward(norm2(h)).
    mixer / feed_forward are any registered spec objects with a `kind`."""
    kind: str
    norm1: object
    mixer: object
    norm2: object
    feed_forward: object


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order: run `layer`; if `cache_from` names another layer, this
    run reads that layer's cache and writes none of its own."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    """kind "lookup": residual stream row = table row of the token id, widened to float32."""
    weight: str
    vocab_size: int
    dim: int
    kind: str = "lookup"


@dataclass(frozen=True)
class HeadSpec:
    """kind "linear": logits = x . W^T in float32, no bias, for the wanted rows only."""
    weight: str  # the embedding's name when input and output embeddings are tied
    vocab_size: int
    dim: int
    kind: str = "linear"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    embedding: object  # any registered "embedding" spec with `kind`, `weight`, `vocab_size`, `dim`
    layers: Tuple[BlockSpec, ...]
    order: Tuple[LayerRun, ...]
    final_norm: object
    head: object       # any registered "head" spec with `kind`, `weight`, `vocab_size`, `dim`
    max_positions: int
    eos_token_ids: FrozenSet[int] = field(default_factory=frozenset)
    # names that may be present in the checkpoint without being read, each with the needed tensor
    # it must agree with in shape (a tied lm_head saved beside the embedding)
    duplicates: Dict[str, str] = field(default_factory=dict)
    # shell-style patterns of names that a checkpoint may carry and nobody reads (buffers that some
    # exporters save, such as "*.rotary_emb.inv_freq"); the reference maps whatever a file holds and
    # reads what it needs (src/weights.cpp:269-301), so it ignores them too
    ignore: Tuple[str, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.head.vocab_size

    @property
    def hidden_size(self) -> int:
        return self.embedding.dim
