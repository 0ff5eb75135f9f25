"""Interfaces of the parts a layer is put together from.

Every part
  * takes its sizes and constants as constructor arguments,
  * declares its parameters with ``params()`` (name -> ParamSpec),
  * receives the loaded tensors with ``bind(tensors, runtime)``,
and does not know which model it is in.  ``Runtime`` carries what all parts share: the
compute type, the device and a workspace of reusable activation buffers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .spec import CacheNeed, ParamSpec


class Workspace:
    """Reusable activation buffers, keyed by a tag, grown on demand and viewed per call.

    Steps run one after another on one stream, so a buffer is free again when the next
    step asks for it.  Shapes depend on the number of tokens in the step only.
    """

    def __init__(self, device: torch.device, keep_outgrown: bool = False):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[Tuple, torch.Tensor] = {}    # (tag, dtype, shape) -> the view handed out last time
        self.frozen = False  # set while a CUDA graph holds pointers into the buffers
        # keep_outgrown: a buffer that has to grow is replaced but stays allocated, because captured
        # graphs hold its address (the workspace that all graphs of a runner share: steps run one after
        # another, so graphs of different shapes can use the same buffers).
        self.keep_outgrown = keep_outgrown
        self._outgrown = []

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in list(self._buffers.values()) + self._outgrown)

    def get(self, tag: str, shape: Tuple[int, ...], dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A view of the buffer ``tag``.  zero: the buffer is zero when it is first made (or
        made larger); its users keep it so."""
        vkey = (tag, dtype, shape)
        v = self._views.get(vkey)
        if v is not None:
            return v
        n = 1
        for s in shape:
            n *= s
        key = (tag, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen and buf is not None:
                raise RuntimeError(f"workspace buffer '{tag}' would move while a graph holds it")
            if self.keep_outgrown and buf is not None:
                self._outgrown.append(buf)
            make = torch.zeros if zero else torch.empty
            buf = make(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            # views of the old buffer are stale
            for k in [k for k in self._views if k[0] == tag and k[1] == dtype]:
                del self._views[k]
        v = buf[:n].view(shape)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[vkey] = v
        return v


@dataclass
class Runtime:
    dtype: torch.dtype          # compute type: torch.float32 or torch.bfloat16
    device: torch.device
    workspace: Workspace

    @property
    def true_fp32(self) -> bool:
        return self.dtype == torch.float32


class Part:
    kind = "?"
    # True if ``forward`` launches the same kernels with the same arguments for every batch of one shape:
    # it reads the step's arrays on the device only (not the host lists q_lens / q_starts /
    # host_state_slots), never waits for the device and allocates through the workspace.  Steps of a
    # model whose parts all say so may be recorded into CUDA graphs.
    graph_safe = False

    def params(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        for k, v in tensors.items():
            setattr(self, "w_" + k.replace(".", "_"), v)

    def launch_plan(self, step) -> None:
        """Makes the launch plans this part will use for ``step`` and leaves them in ``step.plans``
        (key -> plan, both hashable).  The runner calls it on a step context that describes a shape
        and a longest context, without running anything, to tell apart the captured graphs that such
        steps need: steps whose plans are equal replay the same graph.  A part whose launches depend
        on the step's shape alone has nothing to do."""

    def after_load(self) -> None:
        """Called once, after every part of the model has its tensors: the place to lay a
        parameter out anew for a kernel (another order of rows, a padded copy, a descriptor).
        It must not change what the part computes.  (The reference's
        process_weights_after_loading, atom/model_loader/loader.py:354-360.)"""


# What a mixer or a feed-forward may say about itself, beside its interface (both default to False; the
# arrangement asks before it uses either, so a part that says nothing gets and gives plain tensors):
#   takes_scaled_rows  x may come as parts.linear.ScaledRows (rows whose RMSNorm the part's first product
#                      finishes; ``linear`` and ``gated_linear`` take them as they take a tensor);
#   defers_output      ``forward`` takes the keyword ``defer``; with defer=True it may return its last
#                      product unrun, as a parts.linear.PendingProduct.
# A norm that says ``fuses_products`` takes a PendingProduct as delta and the keyword ``scaled_ok``
# (the receiver of its rows takes ScaledRows).


class Norm(Part):
    """``add_norm``: residual (+= delta), returns the normalised rows in the compute type."""

    fuses_products = False

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], tag: str,
                 rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Encodes positions into queries and keys.  Two forms, a kind chooses one:

    * a table of angles: ``table(rt)`` gives [rows, rotary_dim] float32 (cos of every pair's angle,
      then sin) and ``rows_of(step)`` the table row of every token of the step (the token's position
      unless the kind says otherwise: an offset per request, a position that is not the index in the
      sequence).  The mixer hands both to its fused kernel.
    * anything else: ``table`` gives None and ``apply(q, k, step)`` changes the normalised queries
      [T, heads, head] and keys [T, kv heads, head] in place, between the mixer's norm and its
      cache write.
    """

    rotary_dim = 0

    def table(self, rt: Runtime) -> Optional[torch.Tensor]:
        return None

    def rows_of(self, step) -> torch.Tensor:
        return step.positions

    def apply(self, q: torch.Tensor, k: torch.Tensor, step) -> None:
        """Only called when ``table`` gives None.  The default encodes nothing."""


class Mixer(Part):
    """Mixes information along the sequence.  ``cache_need`` says what it keeps per request.

    State kept in a slot (``cache_need`` of kind "state") is all zeros when a request brings its first
    token: the storage clears the slot at admission, also for a preempted request that is computed
    again.  Pages are not cleared; a mixer reads only positions its request has written."""

    takes_scaled_rows = False
    defers_output = False

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, x: torch.Tensor, step, cache, writes_cache: bool) -> torch.Tensor:
        """x: [T, hidden] normalised input.  ``step`` is the StepContext of this batch,
        ``cache`` the view of this run entry's cache slot.  Returns [T, hidden]."""
        raise NotImplementedError


class FeedForward(Part):
    takes_scaled_rows = False
    defers_output = False

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError
