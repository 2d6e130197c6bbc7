"""Loads the compiled host runtime (C++: cache manager, step batch builder, scheduler core)."""
from __future__ import annotations

import importlib.util
import sys

from ..csrc import build as _build

_MODULE = None


def host_module():
    """The pybind11 module `_llmengine_host`, compiled at first use."""
    global _MODULE
    if _MODULE is None:
        path = _build.host_module_path()
        spec = importlib.util.spec_from_file_location("_llmengine_host", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules.setdefault("_llmengine_host", mod)
        _MODULE = mod
    return _MODULE
