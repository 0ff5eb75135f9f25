"""Matrix product y = x W^T (+ b) with weights [out, in], as atom/model_ops/linear.py:946-965.

bfloat16: the GEMM library, as the reference does (tgemm.mm, linear.py:960), with 32-bit
accumulation.  float32: the framework's own FMA kernel, never a reduced-precision mode.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import native


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ weight[N, K]^T (+ bias).  ``out`` may be float32 for bf16 operands."""
    if x.dtype == torch.float32:
        b = bias
        if b is not None and b.dtype != torch.float32:
            b = b.float()
        native.gemm_f32(out, x, weight, b)
    else:
        native.gemm_bf16(out, x, weight)
        if bias is not None:
            native.add_bias(out, bias)
    return out
