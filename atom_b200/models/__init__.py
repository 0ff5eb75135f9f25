"""Architectures.  Each module registers its name, its config parser and its spec builder."""
from __future__ import annotations

_loaded = False


def _load_builtin() -> None:
    global _loaded
    if not _loaded:
        _loaded = True
        from . import qwen3  # noqa: F401


from .registry import (  # noqa: E402
    Architecture,
    build_model_spec,
    get_architecture,
    register_architecture,
    registered_architectures,
)

__all__ = [
    "Architecture", "build_model_spec", "get_architecture", "register_architecture",
    "registered_architectures",
]
