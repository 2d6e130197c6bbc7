"""What every architecture's configuration shares: the error type and the reading of a model
folder's config.json and generation_config.json. Nothing here knows an architecture."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional


class ConfigError(ValueError):
    """config.json is missing a key, or its values do not fit together."""


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    with open(path) as f:
        return json.load(f)


def read_generation_config_json(model_dir: str) -> Optional[Dict[str, Any]]:
    """The folder's generation_config.json, whose `eos_token_id` the reference adds to config.json's
    (src/weights.cpp:98-118); None if there is none."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return None
    with open(path) as f:
        return json.load(f)
