"""RMSNorm fused with the residual add (atom/model_ops/layernorm.py:57-75):
   r = x + r;  y = r * rsqrt(mean(r^2) + eps) * w,  computed in 32-bit on a 32-bit residual."""
from __future__ import annotations

from typing import Dict

from .. import native
from .base import Norm
from .registry import register
from .spec import ParamSpec


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float):
        self.size, self.eps = size, eps

    def params(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), role="vector", init="norm")}

    def add_norm(self, residual, delta, tag, rows=None, n_rows=None):
        n = residual.shape[0] if rows is None else (rows.numel() if n_rows is None else n_rows)
        out = self.rt.workspace.get(tag, (n, self.size), self.rt.dtype)
        native.add_rmsnorm(out, residual, delta, self.w_weight, self.eps, rows, n)
        return out
