"""Typed configurations and the registry from an architecture's name to its model."""
from .files import ConfigError, read_config_json, read_generation_config_json
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, architecture_names, config_from_dir, get_architecture,
                       register_architecture)

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "read_config_json", "read_generation_config_json",
           "Architecture", "architecture_names", "config_from_dir", "get_architecture",
           "register_architecture"]
