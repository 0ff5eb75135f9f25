"""Data that describes a model: parts, their parameters, the layers and their run order.

An architecture (``atom_b200/models/<name>.py``) turns its typed configuration into a
``ModelSpec``.  The spec is plain data: which mixer, feed-forward, norm and position
encoding each layer has, with the sizes and constants each takes as arguments, from which
checkpoint tensors each parameter is read, and the order in which layers run.  Nothing in
the engine, the cache manager or the loader knows an architecture by name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class ParamSpec:
    """One parameter tensor of a part.

    role   "matrix": operand of a matrix product, held in the engine's compute type.
           "vector": norm weight or bias; held in bfloat16 unless stored (or run) in 32-bit.
           "table":  integer table, held as int32.
    init   distribution of the random-weights mode: "normal" N(0, 0.02^2), "norm" U(0.8, 1.2),
           "zeros".
    rows   when the parameter is several checkpoint tensors stacked along dim 0, their row counts.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    rows: Optional[Tuple[int, ...]] = None


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by registry key with its constructor arguments.

    sources maps a parameter name of the part to the checkpoint tensor names it is read
    from (more than one: stacked along dim 0 in that order).  A parameter absent from
    ``sources`` is not read from the checkpoint (e.g. a tied output matrix).
    """

    kind: str
    args: Dict[str, Any] = field(default_factory=dict)
    sources: Dict[str, Tuple[str, ...]] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer and a feed-forward, each behind its norm, in a named arrangement."""

    arrangement: str
    mixer_norm: PartSpec
    mixer: PartSpec
    ffn_norm: PartSpec
    ffn: PartSpec


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: run layer ``layer`` on cache ``cache``.

    A layer may be named by several entries (its weights are shared); ``cache`` names the
    cache slot the mixer uses, and with ``writes_cache=False`` the mixer only reads what
    another entry wrote to that slot in the same step.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    # Regular expressions of checkpoint tensor names that are neither read nor reported.
    ignored_tensors: Tuple[str, ...] = ()
    # (name, other): a checkpoint tensor that the model does not read but that may be present when it
    # is, element for element, the tensor ``other``; present and different is a loading error.
    duplicate_tensors: Tuple[Tuple[str, str], ...] = ()
    eos_token_ids: Tuple[int, ...] = ()


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per request between steps.

    kind "pages": keys and values of every position (or of the last ``window`` positions),
                  num_kv_heads x head_dim each, held in pages.
    kind "state": one array of fixed shape per request, held in a slot.
    """

    kind: str
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"

    def group_key(self) -> Tuple:
        if self.kind == "pages":
            return ("pages", self.num_kv_heads, self.head_dim, self.window)
        return ("state", self.state_shape, self.state_dtype)
