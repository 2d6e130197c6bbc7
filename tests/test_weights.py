"""Safetensors reading, the one error that lists everything wrong, random-weights mode (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import llmengine
from llmengine.config import LlamaConfig
from llmengine.models.llama import describe_llama
from llmengine.weights import (Checkpoint, SafetensorsError, SafetensorsFile, WeightError, load_tensors,
                               model_tensor_needs, random_tensors, write_random_model, write_safetensors)
from tiny import TINY_A, TINY_B

CPU = torch.device("cpu")


def _load(d, cfg, dtype=torch.float32):
    spec = describe_llama(LlamaConfig.from_dict(cfg))
    return load_tensors(Checkpoint(str(d)), model_tensor_needs(spec), spec.duplicates, CPU, dtype)


def test_random_model_round_trip_and_precisions(tmp_path):
    write_random_model(str(tmp_path), TINY_B, seed=4, dtype=torch.bfloat16)
    assert sorted(os.listdir(tmp_path)) == ["config.json", "model.safetensors"]
    t = _load(tmp_path, TINY_B, torch.bfloat16)
    assert "lm_head.weight" not in t  # tied: the head is the embedding
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16 and t["model.embed_tokens.weight"].shape == (509, 192)
    assert t["model.layers.2.self_attn.k_proj.weight"].shape == (32, 192)
    assert t["model.norm.weight"].dtype == torch.float32  # vectors are always float32
    assert abs(float(t["model.norm.weight"].mean()) - 1.0) < 0.05
    assert abs(float(t["model.layers.0.mlp.down_proj.weight"].float().std()) - 0.02) < 0.003
    t32 = _load(tmp_path, TINY_B, torch.float32)  # the 32-bit path widens exactly
    assert torch.equal(t32["model.layers.1.mlp.up_proj.weight"], t["model.layers.1.mlp.up_proj.weight"].float())


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    spec_a = describe_llama(LlamaConfig.from_dict(TINY_A))
    one = random_tensors(spec_a, 7, torch.float32)
    two = random_tensors(spec_a, 7, torch.float32)
    other = random_tensors(spec_a, 8, torch.float32)
    assert all(torch.equal(one[k], two[k]) for k in one)
    assert not torch.equal(one["model.norm.weight"], other["model.norm.weight"])
    # a tensor's values do not depend on which other tensors the model has
    more_layers = describe_llama(LlamaConfig.from_dict(dict(TINY_A, num_hidden_layers=3)))
    assert torch.equal(random_tensors(more_layers, 7, torch.float32)["model.layers.1.mlp.up_proj.weight"],
                       one["model.layers.1.mlp.up_proj.weight"])


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    spec = describe_llama(LlamaConfig.from_dict(TINY_A))
    t = random_tensors(spec, 1, torch.float32)
    del t["model.layers.0.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.1.self_attn.k_proj.weight"] = t["model.layers.1.self_attn.k_proj.weight"].t().contiguous()
    t["model.layers.9.extra.weight"] = torch.zeros(3)
    t["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(TINY_A, f)
    with pytest.raises(WeightError) as e:
        _load(tmp_path, TINY_A)
    err = e.value
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert len(err.wrong) == 2
    msg = str(err)
    assert "k_proj.weight: expected [32, 64], got [64, 32]" in msg and "input_layernorm.weight: expected a floating-point" in msg
    assert "missing tensors (2)" in msg and "unexpected tensors (1)" in msg


def test_tied_head_saved_beside_embedding(tmp_path):
    spec = describe_llama(LlamaConfig.from_dict(TINY_B))
    t = random_tensors(spec, 1, torch.float32)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    loaded = _load(tmp_path, TINY_B)  # accepted and not read
    assert "lm_head.weight" not in loaded
    t["lm_head.weight"] = torch.zeros(5, 192)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightError, match="tied to model.embed_tokens.weight"):
        _load(tmp_path, TINY_B)
    # untied model: lm_head is its own tensor
    a = _load_untied(tmp_path)
    assert a["lm_head.weight"].data_ptr() != a["model.embed_tokens.weight"].data_ptr()


def _load_untied(tmp_path):
    d = tmp_path / "untied"
    write_random_model(str(d), TINY_A, seed=2, dtype=torch.float32)
    return _load(d, TINY_A)


def _raw_file(path, header: dict, data: bytes, header_len=None):
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj) if header_len is None else header_len))
        f.write(hj)
        f.write(data)


def test_malformed_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    with open(p, "wb") as f:
        f.write(b"abc")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsFile(p)
    _raw_file(p, {}, b"", header_len=10 ** 9)
    with pytest.raises(SafetensorsError, match="header overruns"):
        SafetensorsFile(p)
    _raw_file(p, {"w": {"dtype": "F32", "shape": [2, -1], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="negative shape"):
        SafetensorsFile(p)
    _raw_file(p, {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="offsets out of range"):
        SafetensorsFile(p)
    _raw_file(p, {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="byte-count mismatch"):
        SafetensorsFile(p)
    _raw_file(p, {"w": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="unsupported safetensors dtype"):
        SafetensorsFile(p)
    os.remove(p)
    with pytest.raises(SafetensorsError, match="no .safetensors files"):
        Checkpoint(str(tmp_path))


def test_reader_agrees_with_the_safetensors_library(tmp_path):
    from safetensors.numpy import save_file
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = np.arange(5, dtype=np.int32)
    save_file({"a": a, "b": b}, str(tmp_path / "m.safetensors"))
    f = SafetensorsFile(str(tmp_path / "m.safetensors"))
    assert f.names() == ["a", "b"]
    np.testing.assert_array_equal(f.tensor("a").numpy(), a)
    assert f.tensor("b").dtype == torch.int32 and f.tensor("b").tolist() == b.tolist()


def test_engine_validates_inputs_before_reading_weights(tmp_path):
    """Input errors come before weight errors (src/engine.cpp:720-728)."""
    from cpu_ops import CpuOps
    with open(tmp_path / "config.json", "w") as f:
        json.dump(TINY_A, f)
    write_safetensors(str(tmp_path / "model.safetensors"), {"model.norm.weight": torch.ones(64)})
    eng = llmengine.Engine(str(tmp_path), "fp32", device="cpu", ops=CpuOps())
    assert eng.has_weight("model.norm.weight") and not eng.has_weight("lm_head.weight")
    with pytest.raises(ValueError, match="empty"):
        eng.generate([], 3)
    with pytest.raises(ValueError, match="negative"):
        eng.generate([1], -1)
    with pytest.raises(ValueError, match="out of range"):
        eng.generate([1, 256], 3)
    with pytest.raises(RuntimeError, match="position limit"):
        eng.generate([1] * 100, 29)
    with pytest.raises(WeightError, match="missing tensors"):
        eng.generate([1, 2], 3)
    with pytest.raises(ValueError, match="dtype must be"):
        llmengine.Engine(str(tmp_path), "int8", device="cpu", ops=CpuOps())
