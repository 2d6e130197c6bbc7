"""Configuration parsing and the architecture registry (no GPU)."""
import json

import pytest

from llmengine.config import (ConfigError, LlamaConfig, architecture_names, config_from_dir,
                              get_architecture, register_architecture)
from llmengine.models.llama import describe_llama
from tiny import TINY_A, TINY_B


def test_llama_keys_and_defaults():
    c = LlamaConfig.from_dict(TINY_A)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (64, 176, 2)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (4, 2, 16)
    assert c.vocab_size == 256 and c.max_position_embeddings == 128 and c.max_pos == 128
    assert abs(c.rms_norm_eps - 1e-6) < 1e-12 and c.rope_theta == 10000.0
    assert not c.tie_word_embeddings and not c.rope_has_scaling and c.eos_token_ids == frozenset()
    # defaults of the reference's load_config: kv heads = heads, head_dim = hidden/heads, eps 1e-5, theta 1e4
    d = dict(TINY_A)
    for k in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta"):
        d.pop(k)
    c2 = LlamaConfig.from_dict(d)
    assert c2.num_key_value_heads == 4 and c2.head_dim == 16 and c2.rope_theta == 10000.0
    assert abs(c2.rms_norm_eps - 1e-5) < 1e-10


def test_llama3_scaling_both_layouts_and_eos_merge():
    c = LlamaConfig.from_dict(TINY_B, {"eos_token_id": [7, 9]})
    s = c.rope_scaling
    assert (s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings) == (8.0, 1.0, 4.0, 64)
    assert c.rope_has_scaling and c.rope_factor == 8.0 and c.rope_original_max_pos == 64
    assert c.eos_token_ids == frozenset({7, 9}) and c.tie_word_embeddings
    d = dict(TINY_B)
    rs = d.pop("rope_scaling")
    d["rope_parameters"] = dict(rs, rope_theta=250000.0)
    d["eos_token_id"] = 3
    c2 = LlamaConfig.from_dict(d, {"eos_token_id": [7]})
    assert c2.rope_theta == 250000.0 and c2.rope_scaling == s and c2.eos_token_ids == frozenset({3, 7})
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": 1234.0}
    c3 = LlamaConfig.from_dict(d)
    assert c3.rope_scaling is None and c3.rope_theta == 1234.0
    # a rope_scaling block without a type is read as llama3, as the reference does
    d2 = dict(TINY_B, rope_scaling={k: v for k, v in rs.items() if k != "rope_type"})
    assert LlamaConfig.from_dict(d2).rope_scaling == s


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"hidden_size": 0}, "hidden_size"),
    ({"vocab_size": None}, "vocab_size"), ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "original_max_position_embeddings"),
    ({"rms_norm_eps": 0.0}, "eps"), ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
])
def test_config_errors(patch, word):
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(dict(TINY_A, **patch))


def test_round_trip_through_json():
    for cfg in (TINY_A, TINY_B):
        c = LlamaConfig.from_dict(cfg)
        assert LlamaConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_registry(tmp_path):
    assert "LlamaForCausalLM" in architecture_names()
    with open(tmp_path / "config.json", "w") as f:
        json.dump(TINY_B, f)
    with open(tmp_path / "generation_config.json", "w") as f:
        json.dump({"eos_token_id": [5]}, f)
    arch, cfg = config_from_dir(str(tmp_path))
    assert arch.name == "LlamaForCausalLM" and cfg.eos_token_ids == frozenset({5})
    with open(tmp_path / "config.json", "w") as f:
        json.dump(dict(TINY_B, architectures=["NoSuchModel"]), f)
    with pytest.raises(ConfigError, match="unknown architecture 'NoSuchModel'"):
        config_from_dir(str(tmp_path))
    with pytest.raises(ValueError, match="already registered"):
        register_architecture(get_architecture("LlamaForCausalLM"))
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_dir(str(tmp_path / "nowhere"))


def test_description_follows_the_configuration():
    """No size stands in code: every number of the description comes from config.json."""
    for cfg in (TINY_A, TINY_B):
        c = LlamaConfig.from_dict(cfg)
        spec = describe_llama(c)
        assert len(spec.layers) == c.num_hidden_layers == len(spec.order)
        assert [r.layer for r in spec.order] == list(range(c.num_hidden_layers))
        b = spec.layers[-1]
        assert (b.mixer.num_heads, b.mixer.num_kv_heads, b.mixer.head_dim) == (c.num_attention_heads, c.num_key_value_heads, c.head_dim)
        assert b.feed_forward.intermediate == c.intermediate_size and b.norm1.eps == c.rms_norm_eps
        assert b.mixer.position.theta == c.rope_theta and b.mixer.position.max_positions == c.max_position_embeddings
        assert spec.head.weight == ("model.embed_tokens.weight" if c.tie_word_embeddings else "lm_head.weight")
        assert spec.vocab_size == c.vocab_size and spec.max_positions == c.max_position_embeddings
