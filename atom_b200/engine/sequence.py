"""One request's state on the host (after atom/model_engine/sequence.py:40-281): its tokens
(prompt, then what was generated), how many of them are in the cache, status and timing."""
from __future__ import annotations

import enum
import time
from typing import List, Optional

from ..sampling.params import SamplingParams


class SequenceStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class Sequence:
    def __init__(self, prompt_token_ids: List[int], params: SamplingParams, seq_id: int,
                 stop_token_sequences: Optional[List[List[int]]] = None, sibling_index: int = 0):
        # The id comes from whoever owns the request (an engine counts its own requests from 0): it
        # feeds the default random seed, so it must not depend on what else ran in the process.
        self.seq_id = seq_id
        self.token_ids: List[int] = list(prompt_token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        self.params = params
        self.status = SequenceStatus.WAITING
        self.num_computed = 0            # tokens whose keys/values are in the cache
        self.finish_reason: Optional[str] = None
        self.num_preemptions = 0
        self.arrive_time = time.perf_counter()
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.stop_token_sequences: List[List[int]] = [list(x) for x in (stop_token_sequences or []) if x]
        self.sibling_index = sibling_index        # which of the n completions of one prompt this is
        self.return_logprobs = bool(params.logprobs)
        self.logprobs: List[float] = []           # of every generated token, if asked for

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def output_token_ids(self) -> List[int]:
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def num_output_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def num_uncomputed(self) -> int:
        return len(self.token_ids) - self.num_computed

    @property
    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED

    def append_token(self, token: int) -> None:
        self.token_ids.append(int(token))
        if self.first_token_time is None:
            self.first_token_time = time.perf_counter()
