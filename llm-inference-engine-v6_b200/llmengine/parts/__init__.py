"""Parts a layer is put together from: mixers, feed-forwards, norms, position encodings, blocks."""
from . import attention, block, embedding, mlp, norm, position  # noqa: F401  (registers the built-in parts)
from .base import (Block, BuildEnv, Embedding, FeedForward, Head, KVNeed, LayerCache, Mixer, Norm, NormalizedRows,
                   Part, PositionEncoding, Residual, StateNeed)
from .registry import build_part, part_class, register_part
from .spec import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerRun, ModelSpec, NormSpec,
                   PositionSpec, TensorNeed)

__all__ = ["Block", "BuildEnv", "Embedding", "FeedForward", "Head", "KVNeed", "LayerCache", "Mixer", "Norm", "NormalizedRows", "Part", "PositionEncoding",
           "Residual", "StateNeed", "build_part", "part_class", "register_part", "AttentionSpec", "BlockSpec",
           "EmbeddingSpec", "GatedMLPSpec", "HeadSpec", "LayerRun", "ModelSpec", "NormSpec", "PositionSpec",
           "TensorNeed"]
