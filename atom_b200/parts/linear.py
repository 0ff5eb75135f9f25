"""Matrix product y = x W^T (+ b) with weights [out, in], as atom/model_ops/linear.py:946-965.

bfloat16: for many rows the GEMM library, as the reference does (tgemm.mm, linear.py:960); for
few rows (decode: up to ``native.ROWS_M`` = 16, K a multiple of 64) the framework's weight-streaming
kernel, which shares out rows of W among the CTAs (``native.gemm_rows``); the gated product of a
long prompt portion on the framework's tcgen05 kernel with the activation in its epilogue
(``native.gemm_pairs``).  All accumulate in 32-bit.  float32: the framework's own FMA kernel, never
a reduced-precision mode.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import native


class PendingProduct:
    """A product out = x W^T (+ bias) of a step with few rows that has been described but not launched.
    A part hands it on in place of its output where the receiver may fold it into a kernel of its
    own (the norm that follows adds it to the residual stream in the product's epilogue); whoever
    cannot use it calls ``run()`` and has the tensor."""
    __slots__ = ("x", "weight", "bias", "out")

    def __init__(self, x, weight, bias, out):
        self.x, self.weight, self.bias, self.out = x, weight, bias, out

    def run(self) -> torch.Tensor:
        return linear(self.x, self.weight, self.bias, self.out)


class ScaledRows:
    """Rows x = bf16(r * w) of a residual stream r whose RMSNorm the next product finishes:
    RMSNorm(r; w) W^T = rstd(r) * (x W^T), with rstd from the sums of squares ``ssq`` [parts, 16] of r's
    ``size`` columns.  ``linear`` and ``gated_linear`` take it as their x."""
    __slots__ = ("x", "ssq", "size", "eps")

    def __init__(self, x, ssq, size, eps):
        self.x, self.ssq, self.size, self.eps = x, ssq, size, eps

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype


def resolve(delta):
    """The tensor of a part's output, whether it came as one or as a product still to run."""
    return delta.run() if isinstance(delta, PendingProduct) else delta


def may_defer(x, weight) -> bool:
    """Whether out = x W^T is a product that a residual epilogue can take (few rows of bf16, sizes the
    row-sharing kernel takes)."""
    if not FOLD_NORMS or isinstance(x, ScaledRows) or x.dtype != torch.bfloat16:
        return False
    return streams(x.shape[0], weight.shape[0], x.shape[1], x.stride(0))


FOLD_NORMS = True     # False: every norm runs as a kernel of its own (for measurements and tests)


def streams(M: int, N: int, K: int, lda: int, gated: bool = False) -> bool:
    """Whether x[M, K] W[N, K]^T (W of 2N rows if gated) runs on the weight-streaming kernel: up to
    ``native.ROWS_M`` rows of sizes it takes.  From 9 rows on only where a CTA's rows make at most eight
    sub-slabs: every sub-slab reads X again, and with the second token tile's shallower ring the library
    wins on a matrix as tall as the head's (measured: 223 against 195 us at 16 rows)."""
    if M > native.ROWS_M or not native.gemm_rows_supports(M, N, K, lda):
        return False
    if M > 8:
        per_cta = -(-N // native.gemm_rows_grid())
        return per_cta <= 8 * (32 if gated else 64)
    return True


PAIRS_MIN_ROWS = 600      # the gated product runs on native.gemm_pairs from this many rows on (0: never)
PAIRS_MIN_FILL = 0.76     # ... where its tiles fill the device's waves at least this well


def pairs_pay(M: int, N: int, K: int, lda: int, ldc: int) -> bool:
    """Whether silu(x gate^T) * (x up^T) of M rows, N outputs runs on the tcgen05 kernel with the activation
    in its epilogue: measured against the library's product plus the activation kernel it wins from 640 rows
    on (not at 512) wherever the tiles (256 rows x 256 outputs, one pair of CTAs each) fill three quarters of
    the device's waves."""
    if PAIRS_MIN_ROWS <= 0 or M < PAIRS_MIN_ROWS or not native.gemm_pairs_supports(M, N, K, lda, ldc):
        return False
    return native.gemm_pairs_waves(M, N, True) >= PAIRS_MIN_FILL


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ weight[N, K]^T (+ bias).  ``out`` may be float32 for bf16 operands."""
    if isinstance(x, ScaledRows):
        native.gemm_rows(x.x, weight, out, bias, ssq_in=x.ssq, norm_size=x.size, norm_eps=x.eps)
        return out
    if x.dtype == torch.float32:
        b = bias
        if b is not None and b.dtype != torch.float32:
            b = b.float()
        native.gemm_f32(out, x, weight, b)
    elif streams(x.shape[0], weight.shape[0], x.shape[1], x.stride(0)):
        native.gemm_rows(x, weight, out, bias)            # few rows: the product is a read of W
    else:
        native.gemm_bf16(out, x, weight)
        if bias is not None:
            native.add_bias(out, bias)
    return out


def gated_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, scratch) -> torch.Tensor:
    """out[M, I] = silu(x W_gate^T) * (x W_up^T) for weight [2I, K] = [gate ; up].  Few rows, and
    long portions in bf16 (``pairs_pay``): one kernel, the activation fused into the product.  Else
    the product into ``scratch(M, 2I)`` and the activation kernel."""
    M, K = x.shape
    I = weight.shape[0] // 2
    if isinstance(x, ScaledRows):
        native.gemm_rows(x.x, weight, out, gated=True, ssq_in=x.ssq, norm_size=x.size, norm_eps=x.eps)
        return out
    if x.dtype == torch.bfloat16 and streams(M, I, K, x.stride(0), gated=True):
        native.gemm_rows(x, weight, out, gated=True)
        return out
    if x.dtype == torch.bfloat16 and pairs_pay(M, I, K, x.stride(0), out.stride(0)):
        native.gemm_pairs(x, weight, out, gated=True)
        return out
    gu = linear(x, weight, None, scratch(M, 2 * I))
    native.silu_mul(out, gu)
    return out
