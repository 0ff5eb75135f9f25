"""SiLU-gated feed-forward (atom/models/qwen3.py:166-198, atom/model_ops/activation.py:78-82):
   gu = x W_gate_up^T;  f = silu(gu[:, :I]) * gu[:, I:];  y = f W_down^T."""
from __future__ import annotations

from typing import Dict

from .base import FeedForward
from .linear import PendingProduct, gated_linear, linear, may_defer
from .registry import register
from .spec import ParamSpec


@register("ffn", "gated_silu")
class GatedSiluMLP(FeedForward):
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the first product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the last product on unrun

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    def params(self) -> Dict[str, ParamSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return {
            "gate_up.weight": ParamSpec((2 * I, H), rows=(I, I)),
            "down.weight": ParamSpec((H, I)),
        }

    def forward(self, x, step, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        f = gated_linear(x, self.w_gate_up_weight, ws.get("ffn.act", (T, self.intermediate_size), dt),
                         lambda m, n: ws.get("ffn.gate_up", (m, n), dt))
        out = ws.get("ffn.out", (T, self.hidden_size), dt)
        if defer and may_defer(f, self.w_down_weight):
            return PendingProduct(f, self.w_down_weight, None, out)
        return linear(f, self.w_down_weight, None, out)
