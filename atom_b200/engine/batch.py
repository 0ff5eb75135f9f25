"""One step's batch: the tokens each request brings, flattened, with the small integer
arrays the kernels read (positions, owning request, block tables, rows whose logits are
wanted).  Prompt portions and single decoded tokens lie side by side; a decoded token is
simply a portion of length one.  Replaces the reference's ScheduledBatch plus attention
metadata (atom/model_engine/scheduler.py:331-568, atom/model_ops/attentions/backends.py:374-497)
with one structure that is passed explicitly."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    num_logits_rows: int
    token_ids: torch.Tensor            # [T] int32
    positions: torch.Tensor            # [T] int32, position of each token in its request
    seq_of_token: torch.Tensor         # [T] int32, row of the block tables
    cu_q: torch.Tensor                 # [S+1] int32, first token of each request in the batch
    ctx_len: torch.Tensor              # [S] int32, tokens of the request in the cache after this step
    state_slots: torch.Tensor          # [S] int32
    logits_rows: torch.Tensor          # [R] int32, token rows whose logits are wanted
    block_tables: Dict[int, torch.Tensor]   # page group -> [S, P] int32
    status: torch.Tensor               # [1] int32, set by kernels on an accounting fault
    # host copies, for work splitting and for mixers that branch on the batch's shape
    q_lens: List[int] = field(default_factory=list)
    q_starts: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_len: int = 0
    logits_out: Optional[torch.Tensor] = None   # where the head writes, if preallocated
    plans: Dict = field(default_factory=dict)    # launch plans that parts share within the step


def pack_layout(T: int, S: int, R: int, widths: Sequence[int]):
    """Offsets (in int32 elements) of the sections of the packed metadata buffer."""
    off, cur = {}, 0
    for name, n in (("token_ids", T), ("positions", T), ("seq_of_token", T), ("cu_q", S + 1),
                    ("ctx_len", S), ("state_slots", S), ("logits_rows", max(R, 1))):
        off[name] = (cur, n)
        cur += -(-n // 4) * 4   # 16-byte aligned sections
    for gi, w in enumerate(widths):
        off[f"bt{gi}"] = (cur, S * w)
        cur += -(-(S * w) // 4) * 4
    return off, cur
