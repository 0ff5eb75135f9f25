"""Data that describes a model: parts, their parameters, the layers and their run order.

An architecture (``atom_b200/models/<name>.py``) turns its typed configuration into a
``ModelSpec``.  The spec is plain data: which mixer, feed-forward, norm and position
encoding each layer has, with the sizes and constants each takes as arguments, from which
checkpoint tensors each parameter is read, and the order in which layers run.  Nothing in
the engine, the cache manager or the loader knows an architecture by name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class ParamSpec:
    """One parameter tensor of a part.

    role   "matrix": operand of a matrix product, held in the engine's compute type.
           "vector": norm weight or bias; held in bfloat16 unless stored (or run) in 32-bit.
           "table":  integer table, held as int32.
    init   distribution of the random-weights mode: "normal" N(0, 0.02^2), "norm" U(0.8, 1.2),
           "zeros".
    rows   when the parameter is several checkpoint tensors stacked along one axis, their extents
           along it.
    stack_dim   that axis (0: rows under one another, as q/k/v; 1: side by side).
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    rows: Optional[Tuple[int, ...]] = None
    stack_dim: int = 0


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by registry key with its constructor arguments.

    sources maps a parameter name of the part to the checkpoint tensor names it is read
    from (more than one: stacked along the parameter's ``stack_dim`` in that order).  A parameter absent from
    ``sources`` is not read from the checkpoint (e.g. a tied output matrix).
    """

    kind: str
    args: Dict[str, Any] = field(default_factory=dict)
    sources: Dict[str, Tuple[str, ...]] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement and the parts it is put together from, by the names under which the
    arrangement knows them.  Which names there are, and of which category each is, is the
    arrangement's affair (its ``slots``): "prenorm" has mixer_norm, mixer, ffn_norm and ffn; another
    arrangement may have four norms, no feed-forward, or two mixers."""

    arrangement: str
    parts: Mapping[str, PartSpec]

    def __hash__(self):
        return hash((self.arrangement, tuple(sorted(self.parts))))


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
class CacheEntry:
    """One array that a mixer keeps in pages: ``shape`` per token, in the compute type unless
    ``dtype`` names a torch type.  In the page array the token axis stands before the last axis:
    (kv heads, head size) is stored as [pages, kv heads, page size, head size], a single row (r,)
    as [pages, page size, r]."""

    name: str
    shape: Tuple[int, ...]
    dtype: str = "compute"


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per request between steps.

    kind "pages": ``entries`` for every position (or for the last ``window`` positions), held in
                  pages.  Giving ``num_kv_heads`` and ``head_dim`` instead stands for the two
                  entries "k" and "v" of that shape each.
    kind "state": one array of fixed shape per request, held in a slot.
    """

    kind: str
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"
    entries: Tuple[CacheEntry, ...] = ()

    def __post_init__(self):
        if self.kind == "pages" and not self.entries:
            if self.num_kv_heads <= 0 or self.head_dim <= 0:
                raise ValueError("a 'pages' cache need names its entries, or kv heads and head size")
            shape = (self.num_kv_heads, self.head_dim)
            object.__setattr__(self, "entries", (CacheEntry("k", shape), CacheEntry("v", shape)))
        if self.kind == "pages":
            names = [e.name for e in self.entries]
            if len(set(names)) != len(names) or any(not e.shape for e in self.entries):
                raise ValueError(f"cache entries need distinct names and a shape per token: {self.entries}")

    def group_key(self) -> Tuple:
        if self.kind == "pages":
            return ("pages", self.entries, self.window)
        return ("state", self.state_shape, self.state_dtype)
