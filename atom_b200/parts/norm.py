"""RMSNorm fused with the residual add (atom/model_ops/layernorm.py:57-75):
   r = x + r;  y = r * rsqrt(mean(r^2) + eps) * w,  computed in 32-bit on a 32-bit residual.

In a step of few rows the norm can do without a kernel of its own.  If what is to be added comes as
a product still to run (``PendingProduct``) and the receiver of the normalised rows takes
``ScaledRows``, the product runs with the residual epilogue (r += x W^T in 32-bit, bf16(r * w) and the
sums of r^2 written beside it) and the receiver's first product multiplies its rows by rstd:
   RMSNorm(r; w) V^T = rstd(r) * ((r * w) V^T).
The sums and rstd stay 32-bit; what differs from the kernel of its own is where bf16 rounds."""
from __future__ import annotations

from typing import Dict

import torch

from .. import native
from . import linear as _linear
from .base import Norm
from .linear import PendingProduct, ScaledRows
from .registry import register
from .spec import ParamSpec


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float):
        self.size, self.eps = size, eps

    def params(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), role="vector", init="norm")}

    fuses_products = True      # add_norm takes a PendingProduct as delta and the keyword scaled_ok

    def add_norm(self, residual, delta, tag, rows=None, n_rows=None, scaled_ok=False):
        if isinstance(delta, PendingProduct):
            if scaled_ok and rows is None and self._folds(residual, delta):
                M, ws = residual.shape[0], self.rt.workspace
                xw = ws.get(tag + ".scaled", (M, self.size), torch.bfloat16)
                ssq = ws.get(tag + ".ssq", (native.gemm_rows_grid(), 16), torch.float32)
                native.gemm_rows(delta.x, delta.weight, residual=residual, norm_w=self.w_weight, xout=xw, ssq_out=ssq)
                return ScaledRows(xw, ssq, self.size, self.eps)
            delta = delta.run()
        n = residual.shape[0] if rows is None else (rows.numel() if n_rows is None else n_rows)
        out = self.rt.workspace.get(tag, (n, self.size), self.rt.dtype)
        native.add_rmsnorm(out, residual, delta, self.w_weight, self.eps, rows, n)
        return out

    def _folds(self, residual, p: PendingProduct) -> bool:
        """The pending product can run with the residual epilogue, and a product over this norm's
        ``size`` columns can take the rows' factors."""
        M = residual.shape[0]
        return (_linear.FOLD_NORMS and p.bias is None and self.rt.dtype == torch.bfloat16
                and residual.dtype == torch.float32 and residual.is_contiguous()
                and p.weight.shape[0] == self.size and _linear.may_defer(p.x, p.weight)
                and M <= native.ROWS_M and native.gemm_rows_supports(M, 1, self.size, self.size))
