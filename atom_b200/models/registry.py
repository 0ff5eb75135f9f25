"""One registry from an architecture's name (``architectures[0]`` of config.json) to its
typed configuration and its model description, as the reference's
``support_model_arch_dict`` (atom/model_engine/model_runner.py:98-124) maps names to model
classes.  Adding an architecture = one module that calls ``register_architecture``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from ..config.model_config import ConfigError, ModelConfig
from ..parts.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Dict[str, Any]], ModelConfig]
    build_spec: Callable[[ModelConfig], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, build_spec) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, build_spec)


def get_architecture(name: str) -> Architecture:
    from . import _load_builtin

    _load_builtin()
    if name not in _ARCHITECTURES:
        known = ", ".join(sorted(_ARCHITECTURES))
        raise ConfigError(f"config.json: architecture '{name}' is not registered (known: {known})")
    return _ARCHITECTURES[name]


def registered_architectures():
    from . import _load_builtin

    _load_builtin()
    return sorted(_ARCHITECTURES)


def build_model_spec(config: ModelConfig) -> ModelSpec:
    return get_architecture(config.architecture).build_spec(config)
