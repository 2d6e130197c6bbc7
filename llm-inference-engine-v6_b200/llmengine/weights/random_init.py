"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode in C++ (its tests save a seeded model from another library,
tests/fixtures.py:16-55). Here every tensor the model description names is drawn on the CPU from a
generator keyed by (seed, tensor name), so a tensor's values depend on nothing else: not on the
order of tensors, not on the device. What is drawn is a field of the part's own `TensorNeed`
(`init`): N(0, std) by default, N(1, std) for weights that multiply (norm weights), zeros for
additive terms; std defaults to 0.02.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from ..config.registry import get_architecture
from ..parts.registry import part_class
from ..parts.spec import ModelSpec, TensorNeed
from .loader import merge_needs
from .safetensors_io import write_safetensors


def model_tensor_needs(spec: ModelSpec) -> Dict[str, TensorNeed]:
    """Every tensor the described model reads."""
    needs = list(part_class("embedding", spec.embedding.kind).tensor_needs(spec.embedding))
    needs += part_class("head", spec.head.kind).tensor_needs(spec.head)
    for block in spec.layers:
        needs += part_class("block", block.kind).tensor_needs(block)
    needs += part_class("norm", spec.final_norm.kind).tensor_needs(spec.final_norm)
    return merge_needs(needs)


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(spec: ModelSpec, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> Dict[str, torch.Tensor]:
    out = {}
    for name, need in sorted(model_tensor_needs(spec).items()):
        g = torch.Generator(device="cpu")
        g.manual_seed(_tensor_seed(seed, name))
        if need.init == "zeros":
            t = torch.zeros(need.shape, dtype=torch.float32)
        elif need.init in ("normal", "around_one"):
            t = torch.randn(need.shape, generator=g, dtype=torch.float32) * std
            if need.init == "around_one":
                t += 1.0
        else:
            raise ValueError(f"tensor need '{name}': unknown init '{need.init}' (normal, around_one, zeros)")
        out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                       architecture: str = None) -> str:
    """config: a typed configuration (e.g. LlamaConfig) or a config.json dict."""
    if isinstance(config, dict):
        from ..config.registry import architecture_name_of
        arch = get_architecture(architecture or architecture_name_of(config))
        config = arch.parse_config(config, None)
    else:
        arch = get_architecture(architecture or config.architecture)
    spec = arch.describe(config)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(arch.config_to_json(config), f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), random_tensors(spec, seed, dtype, std))
    return model_dir
