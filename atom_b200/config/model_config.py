"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference builds its model from a transformers config object and reads the
keys listed below (atom/models/qwen3.py:213-239, atom/config.py:1690-1753).  Here
``config.json`` is parsed by hand into a frozen dataclass; every size and
constant a layer needs comes from it and nothing is hard-coded elsewhere.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model; names the offending key."""


_MISSING = object()


def cfg_get(d: Dict[str, Any], key: str, typ, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if typ is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if typ is int and isinstance(v, bool):
        raise ConfigError(f"config.json: key '{key}' must be int, got bool")
    if not isinstance(v, typ):
        raise ConfigError(
            f"config.json: key '{key}' must be {typ.__name__}, got {type(v).__name__} ({v!r})"
        )
    return v


def cfg_positive(name: str, v: int) -> int:
    if v <= 0:
        raise ConfigError(f"config.json: key '{name}' must be positive, got {v}")
    return v


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration."""

    architecture: str

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    @property
    def eos_token_ids(self) -> Tuple[int, ...]:
        return ()


def config_from_dict(d: Dict[str, Any]) -> ModelConfig:
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    from atom_b200.models.registry import get_architecture

    return get_architecture(archs[0]).config_from_dict(d)


def load_model_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    gen = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen):
        # The reference takes stop ids from generation_config.json (atom/config.py:1724-1729).
        with open(gen, "r") as f:
            g = json.load(f)
        if isinstance(g, dict) and g.get("eos_token_id") is not None and d.get("eos_token_id") is None:
            d = dict(d)
            d["eos_token_id"] = g["eos_token_id"]
    return config_from_dict(d)


def save_model_config(cfg: ModelConfig, model_dir: str) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f, indent=1, sort_keys=True)
