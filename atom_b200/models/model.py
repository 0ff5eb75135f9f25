"""A model assembled from a ModelSpec: embedding, blocks in their run order, final norm, head.

The class is the same for every architecture; what differs is the spec.  ``forward`` runs
the tokens of one step (any mixture of prompt portions and decoded tokens) and returns
32-bit logits at the rows that were asked for.
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Optional, Tuple

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..parts import registry
from ..parts.base import Part, Runtime
from ..parts.linear import resolve
from ..parts.spec import CacheNeed, ModelSpec, PartSpec


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = registry.build("embedding", spec.embedding)
        self.blocks = []
        self._named: List[Tuple[str, Part, PartSpec]] = [("embedding", self.embedding, spec.embedding)]
        for i, ls in enumerate(spec.layers):
            arrangement = registry.lookup("arrangement", ls.arrangement)
            slots = arrangement.slots          # name -> part category ("norm", "mixer", "ffn", ...)
            absent = [n for n in slots if n not in ls.parts and n not in arrangement.optional]
            extra = [n for n in ls.parts if n not in slots]
            if absent or extra:
                raise ValueError(f"layer {i}: arrangement '{ls.arrangement}' has the parts {sorted(slots)}; "
                                 f"missing {absent}, not known {extra}")
            built = {n: registry.build(slots[n], ls.parts[n]) for n in slots if n in ls.parts}
            self.blocks.append(arrangement(**built))
            self._named += [(f"layers.{i}.{n}", built[n], ls.parts[n]) for n in slots if n in built]
        self.final_norm = registry.build("norm", spec.final_norm)
        self.lm_head = registry.build("head", spec.lm_head)
        self._named += [("final_norm", self.final_norm, spec.final_norm), ("lm_head", self.lm_head, spec.lm_head)]
        for e in spec.run_order:
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"run order names layer {e.layer}, the model has {len(self.blocks)}")
        self.rt: Optional[Runtime] = None

    # ------------------------------------------------------------------ description

    def named_parts(self) -> Iterator[Tuple[str, Part, PartSpec]]:
        return iter(self._named)

    @property
    def graph_safe(self) -> bool:
        """Every part says that its launches depend on a step's shape only (Part.graph_safe)."""
        return all(part.graph_safe for _, part, _ in self._named)

    def cache_needs(self) -> Dict[int, CacheNeed]:
        """Cache slot -> what the mixers that run on it keep there."""
        needs: Dict[int, CacheNeed] = {}
        writers: Dict[int, int] = {}
        for e in self.spec.run_order:
            mixer = getattr(self.blocks[e.layer], "mixer", None)   # a layer may have none
            need = mixer.cache_need() if mixer is not None else None
            if need is None:
                continue
            if e.cache in needs and needs[e.cache] != need:
                raise ValueError(f"cache slot {e.cache} is used by mixers with different needs")
            needs[e.cache] = need
            if e.writes_cache:
                writers[e.cache] = writers.get(e.cache, 0) + 1
        for c in needs:
            if writers.get(c, 0) == 0:
                raise ValueError(f"cache slot {c} is read but never written")
        return needs

    # ------------------------------------------------------------------ weights

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        """tensors: '<part path>.<param name>' -> tensor on the device."""
        self.rt = rt
        for path, part, _ in self._named:
            own = {}
            for name in part.params():
                key = f"{path}.{name}"
                if key not in tensors:
                    raise KeyError(f"parameter {key} was not loaded")
                own[name] = tensors[key]
            part.bind(own, rt)
        if getattr(self.lm_head, "tied", False):
            self.lm_head.tie(self.embedding)
        for _, part, _ in self._named:
            part.after_load()

    def plan_signature(self, step) -> tuple:
        """What the parts' launch plans for ``step`` are, as one hashable value: two steps of one shape
        with equal signatures launch the same kernels with the same arguments."""
        step.plans.clear()
        for _, part, _ in self._named:
            part.launch_plan(step)
        return tuple(sorted(step.plans.items(), key=repr))

    # ------------------------------------------------------------------ compute

    def forward(self, step, caches) -> torch.Tensor:
        """step: StepContext; caches: cache slot -> CacheView.  Returns [R, vocab] float32."""
        residual = self.embedding.forward(step.token_ids, step.num_tokens)
        delta = None
        for e in self.spec.run_order:
            block = self.blocks[e.layer]
            if not getattr(block, "takes_pending", False):
                delta = resolve(delta)      # (a block may hand its last product on unrun)
            delta = block.run(residual, delta, step, caches.get(e.cache), e.writes_cache)
        y = self.final_norm.add_norm(residual, resolve(delta), "norm.final", step.logits_rows, step.num_logits_rows)
        return self.lm_head.forward(y, step.logits_out)
