"""Typed configuration of the Llama dense GQA decoder, read from the architecture's own
config.json keys.

Keys and defaults follow the reference's load_config (src/weights.cpp:55-121) and ModelConfig
(include/llmengine/config.hpp:9-31). Differences, all on purpose:
  * consistency checks the reference lacks (heads divisible by groups, even head size, ...);
  * `rope_type` is checked: only "llama3" (scaled) and "default" (plain) are accepted, where the
    reference treats any `rope_scaling` block as llama3 (src/weights.cpp:94-96);
  * the position limit is `max_position_embeddings`; the reference's cap at
    min(original_max_position_embeddings, 8192) (include/llmengine/config.hpp:39-45) is a limit of
    its table, not of the architecture, and is not kept.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, FrozenSet, Optional

import numpy as np

from .files import ConfigError


def _f32(x) -> float:
    """theta, the factors and eps are `float` fields in the reference; round once, here."""
    return float(np.float32(x))


@dataclass(frozen=True)
class RopeScaling:
    """Llama-3 wavelength-band rescaling of the rotary frequencies (src/kernels.cpp:114-160)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    rope_scaling: Optional[RopeScaling] = None
    eos_token_ids: FrozenSet[int] = field(default_factory=frozenset)

    # ---- names the reference exposes on its ModelConfig binding (src/bindings.cpp:130-148)
    @property
    def rope_has_scaling(self) -> bool:
        return self.rope_scaling is not None

    @property
    def rope_factor(self) -> float:
        return self.rope_scaling.factor if self.rope_scaling else 1.0

    @property
    def rope_low_freq_factor(self) -> float:
        return self.rope_scaling.low_freq_factor if self.rope_scaling else 1.0

    @property
    def rope_high_freq_factor(self) -> float:
        return self.rope_scaling.high_freq_factor if self.rope_scaling else 1.0

    @property
    def rope_original_max_pos(self) -> int:
        return self.rope_scaling.original_max_position_embeddings if self.rope_scaling else 0

    @property
    def max_pos(self) -> int:
        """Largest number of tokens a request may hold."""
        return self.max_position_embeddings

    # ---- parsing
    @staticmethod
    def from_dict(j: Dict[str, Any], generation_config: Optional[Dict[str, Any]] = None) -> "LlamaConfig":
        def need(key: str) -> int:
            if key not in j or j[key] is None:
                raise ConfigError(f"config.json: missing key '{key}'")
            v = j[key]
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"config.json: '{key}' must be a positive integer, got {v!r}")
            return v

        # options the reference never reads, so their meaning is fixed in its code (and in ours):
        # refuse a checkpoint that needs something else instead of running it wrongly
        if j.get("hidden_act", "silu") not in ("silu", "swish"):
            raise ConfigError(f"hidden_act '{j.get('hidden_act')}' is not supported (the feed-forward is SiLU-gated)")
        for key in ("attention_bias", "mlp_bias"):
            if j.get(key):
                raise ConfigError(f"config.json: '{key}' is set, but linear layers with bias are not supported")
        archs = j.get("architectures") or ["LlamaForCausalLM"]
        hidden = need("hidden_size")
        heads = need("num_attention_heads")
        kv_heads = j.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else kv_heads
        head_dim = j.get("head_dim")
        head_dim = hidden // heads if head_dim is None else head_dim

        theta = _f32(j.get("rope_theta", 10000.0))
        scaling = None

        def parse_scaling(rs: Dict[str, Any]) -> RopeScaling:
            orig = rs.get("original_max_position_embeddings", 0)
            if not isinstance(orig, int) or orig <= 0:
                raise ConfigError("rope scaling: 'original_max_position_embeddings' must be a positive integer")
            s = RopeScaling(_f32(rs.get("factor", 1.0)), _f32(rs.get("low_freq_factor", 1.0)),
                            _f32(rs.get("high_freq_factor", 1.0)), orig)
            if s.factor <= 0 or s.low_freq_factor <= 0 or s.high_freq_factor <= 0:
                raise ConfigError("rope scaling: factors must be positive")
            if s.high_freq_factor == s.low_freq_factor:
                raise ConfigError("rope scaling: high_freq_factor must differ from low_freq_factor")
            return s

        def rope_kind(block: Dict[str, Any]) -> str:
            kind = block.get("rope_type", block.get("type", "default"))
            if kind not in ("default", "llama3"):
                raise ConfigError(f"rope_type '{kind}' is not supported (supported: default, llama3)")
            return kind

        # `rope_parameters` (newer layout) wins over `rope_scaling` (src/weights.cpp:87-96)
        if j.get("rope_parameters") is not None:
            rp = j["rope_parameters"]
            theta = _f32(rp.get("rope_theta", theta))
            if rope_kind(rp) == "llama3":
                scaling = parse_scaling(rp)
        elif j.get("rope_scaling") is not None:
            rs = j["rope_scaling"]
            if rope_kind(rs) == "llama3" or "rope_type" not in rs and "type" not in rs:
                scaling = parse_scaling(rs)

        eos = set()

        def absorb(src: Optional[Dict[str, Any]]) -> None:  # src/weights.cpp:98-118
            if not src:
                return
            e = src.get("eos_token_id")
            if isinstance(e, list):
                eos.update(int(v) for v in e)
            elif isinstance(e, int) and not isinstance(e, bool):
                eos.add(e)

        absorb(j)
        absorb(generation_config)

        cfg = LlamaConfig(
            architecture=str(archs[0]),
            hidden_size=hidden,
            intermediate_size=need("intermediate_size"),
            num_hidden_layers=need("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=need("vocab_size"),
            max_position_embeddings=need("max_position_embeddings"),
            rms_norm_eps=_f32(j.get("rms_norm_eps", 1e-5)),
            rope_theta=theta,
            tie_word_embeddings=bool(j.get("tie_word_embeddings", False)),
            rope_scaling=scaling,
            eos_token_ids=frozenset(eos),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for k in ("num_key_value_heads", "head_dim"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"config.json: '{k}' must be a positive integer, got {v!r}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                              f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotary position encoding")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")
        if not (self.rope_theta > 0):
            raise ConfigError("rope_theta must be positive")
        for t in self.eos_token_ids:
            if t < 0:
                raise ConfigError(f"eos_token_id {t} is negative")

    def to_dict(self) -> Dict[str, Any]:
        """config.json content that parses back to this configuration."""
        d: Dict[str, Any] = dict(
            architectures=[self.architecture], model_type="llama",
            hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
            num_hidden_layers=self.num_hidden_layers, num_attention_heads=self.num_attention_heads,
            num_key_value_heads=self.num_key_value_heads, head_dim=self.head_dim,
            vocab_size=self.vocab_size, max_position_embeddings=self.max_position_embeddings,
            rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta,
            tie_word_embeddings=self.tie_word_embeddings,
        )
        if self.rope_scaling is not None:
            s = self.rope_scaling
            d["rope_scaling"] = dict(rope_type="llama3", factor=s.factor, low_freq_factor=s.low_freq_factor,
                                     high_freq_factor=s.high_freq_factor,
                                     original_max_position_embeddings=s.original_max_position_embeddings)
        if self.eos_token_ids:
            d["eos_token_id"] = sorted(self.eos_token_ids)
        return d
