"""Token embedding (atom/model_ops/embed_head.py:177) and output head (:249-252).

The embedding writes the 32-bit residual stream; the head multiplies the normalised rows
whose logits are wanted by the output matrix and returns 32-bit logits.  A tied head uses
the embedding's table (atom/models/qwen3.py:339-340)."""
from __future__ import annotations

from typing import Dict

import torch

from .. import native
from .base import Part
from .linear import linear
from .registry import register
from .spec import ParamSpec


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def params(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def forward(self, token_ids: torch.Tensor, T: int) -> torch.Tensor:
        out = self.rt.workspace.get("residual", (T, self.hidden_size), torch.float32)
        native.embedding(out, self.w_weight, token_ids)
        return out


@register("head", "lm_head")
class LMHead(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool):
        self.vocab_size, self.hidden_size, self.tied = vocab_size, hidden_size, tied

    def params(self) -> Dict[str, ParamSpec]:
        if self.tied:
            return {}
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def tie(self, embedding: TokenEmbedding) -> None:
        self.w_weight = embedding.w_weight

    def forward(self, x: torch.Tensor, out=None) -> torch.Tensor:
        """x: [R, hidden] -> logits [R, vocab] float32; into ``out`` if given, else a fresh
        tensor the caller may keep."""
        if out is None:
            out = torch.empty((x.shape[0], self.vocab_size), dtype=torch.float32, device=x.device)
        return linear(x, self.w_weight, None, out[: x.shape[0]])
