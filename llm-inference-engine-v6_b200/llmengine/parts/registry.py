"""Registry of part classes: (category, kind) -> class.

Categories: "embedding", "norm", "position", "mixer", "feed_forward", "block", "head". A part class is built as
`cls(spec, env)` and must provide the interface of its category (parts/base.py). Registering a
class is all it takes to make a new kind usable from a model description; nothing in the engine
names a concrete part.
"""
from __future__ import annotations

from typing import Dict, Tuple, Type

CATEGORIES = ("embedding", "norm", "position", "mixer", "feed_forward", "block", "head")
_PARTS: Dict[Tuple[str, str], Type] = {}


def register_part(category: str, kind: str, cls: Type, *, replace: bool = False) -> Type:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category '{category}' (one of {', '.join(CATEGORIES)})")
    if (category, kind) in _PARTS and not replace:
        raise ValueError(f"{category} part '{kind}' is already registered")
    _PARTS[(category, kind)] = cls
    return cls


def part_class(category: str, kind: str) -> Type:
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise KeyError(f"no {category} part of kind '{kind}' is registered (registered: {', '.join(known) or 'none'})") from None


def build_part(category: str, spec, env):
    return part_class(category, spec.kind)(spec, env)
