"""Rotary position encoding, half-split pairing ("neox"), as
atom/model_ops/rotary_embedding.py:14-24 (rotation) and :58-80 (table):
   inv_freq_j = 1 / theta^(2j / rotary_dim),  angle = pos * inv_freq_j  (32-bit),
   y1 = x1 cos - x2 sin,  y2 = x2 cos + x1 sin  with x1 = x[:d/2], x2 = x[d/2:].
The table stays in 32-bit in both precisions (the reference casts it to the model type,
:49-50); the rotation itself happens inside the mixer's fused kernel."""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, Runtime
from .registry import register


@register("position", "rope_neox")
class RotaryNeox(PositionEncoding):
    graph_safe = True

    def __init__(self, rotary_dim: int, theta: float, max_position: int):
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        self.rotary_dim, self.theta, self.max_position = rotary_dim, theta, max_position
        self._table: Optional[torch.Tensor] = None

    def table(self, rt: Runtime) -> torch.Tensor:
        """[max_position, rotary_dim] float32: cos of every pair's angle, then sin."""
        if self._table is None or self._table.device != rt.device:
            d = self.rotary_dim
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
            t = torch.arange(self.max_position, dtype=torch.float32)
            ang = torch.outer(t, inv_freq)
            self._table = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous().to(rt.device)
        return self._table


@register("position", "none")
class NoPosition(PositionEncoding):
    graph_safe = True

    def __init__(self):
        pass
