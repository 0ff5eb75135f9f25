"""Per-request sampling options, with the reference's names, defaults and checks
(atom/sampling_params.py:8-30): temperature 1.0 (0 = greedy), top_k -1 (off), top_p 1.0
(off), max_tokens 64, ignore_eos, stop_strings, n (independently sampled completions of one
prompt), logprobs (the log-probability of every sampled token).  Added here: ``seed`` (the
request's own random stream, so that its tokens do not depend on what else is in the batch;
sibling i of n uses seed + i) and ``stop_token_ids``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Union


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False
    stop_strings: Optional[List[str]] = None
    n: int = 1
    logprobs: Optional[Union[bool, int]] = None
    stop_token_ids: List[int] = field(default_factory=list)
    seed: Optional[int] = None

    def __post_init__(self):
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if self.top_k != -1 and self.top_k < 1:
            raise ValueError("top_k must be -1 (disabled) or >= 1")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in range (0.0, 1.0]")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.n < 1:
            raise ValueError("n must be >= 1")
        if isinstance(self.stop_strings, str):
            self.stop_strings = [self.stop_strings]

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def filters(self) -> bool:
        return self.top_k != -1 or self.top_p < 1.0
