"""One registry: architecture name (config.json `architectures[0]`) -> how to parse its
configuration and how to describe its model.

The reference never reads `architectures` (it runs one hard-wired model, src/engine.cpp); here the
name chooses everything, so a second architecture is one more `register_architecture` call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

from .files import ConfigError, read_config_json, read_generation_config_json


@dataclass(frozen=True)
class Architecture:
    """name: value of config.json `architectures[0]`.
    parse_config(config_json, generation_config_json|None) -> typed configuration.
    describe(config) -> parts.spec.ModelSpec (layers, their order, the tensors they need).
    config_to_json(config) -> dict written as config.json by the random-weights mode."""
    name: str
    parse_config: Callable[[Dict[str, Any], Optional[Dict[str, Any]]], Any]
    describe: Callable[[Any], Any]
    config_to_json: Callable[[Any], Dict[str, Any]]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{arch.name}' is already registered")
    _ARCHITECTURES[arch.name] = arch


def architecture_names() -> List[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture '{name}'; registered: {', '.join(architecture_names()) or 'none'}") from None


def architecture_name_of(config_json: Dict[str, Any]) -> str:
    archs = config_json.get("architectures")
    if not archs:
        raise ConfigError("config.json: missing key 'architectures'")
    if not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a list of names")
    return archs[0]


def config_from_dir(model_dir: str):
    """-> (Architecture, typed configuration) for the model folder."""
    j = read_config_json(model_dir)
    arch = get_architecture(architecture_name_of(j))
    return arch, arch.parse_config(j, read_generation_config_json(model_dir))
