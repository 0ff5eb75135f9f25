"""Registries of part classes by kind: mixers, feed-forwards, norms, position encodings,
embeddings, output heads and layer arrangements.  A new part is one class and one
``register`` call; specs name parts by these keys."""
from __future__ import annotations

from typing import Callable, Dict

_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {},
    "ffn": {},
    "norm": {},
    "position": {},
    "embedding": {},
    "head": {},
    "arrangement": {},
}


def register(category: str, kind: str):
    """Class decorator: ``@register("mixer", "paged_attention")``."""
    if category not in _REGISTRIES:
        raise KeyError(f"unknown part category '{category}' (have {sorted(_REGISTRIES)})")

    def deco(cls):
        _REGISTRIES[category][kind] = cls
        cls.kind = kind
        return cls

    return deco


def lookup(category: str, kind: str):
    try:
        return _REGISTRIES[category][kind]
    except KeyError:
        have = ", ".join(sorted(_REGISTRIES.get(category, {})))
        raise KeyError(f"no {category} part registered as '{kind}' (have: {have})") from None


def build(category: str, spec, **extra):
    """Instantiates the part a PartSpec names."""
    return lookup(category, spec.kind)(**spec.args, **extra)
