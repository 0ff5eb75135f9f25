"""The scheduler: admits requests, cuts prompts into portions under a token budget, lets every
running request decode, finishes and frees.

One step may hold decoded tokens of some requests beside prompt portions of others (the
reference schedules either the one or the other, atom/model_engine/scheduler.py:1370-1429).
Order within a step, all charged to one budget of ``max_num_batched_tokens``:
  1. requests that are decoding, one token each, oldest first;
  2. requests in the middle of their prompt, the next portion each;
  3. waiting requests, first come first served, while a place and budget are left.
A portion is min(what is left of the prompt, the per-request cap, the budget left): no
alignment is asked for, down to a single token.

When pages run out:
  * a waiting request is admitted only if, at that moment, every page group has free the
    most pages the request will ever hold; otherwise it waits and nothing behind it is
    admitted (first come, first served);
  * a running request that needs a page and finds none takes it from the NEWEST running
    request (preemption by recomputation, atom/model_engine/scheduler.py:1917-1952): the victim
    gives all its pages back, keeps its tokens and goes to the FRONT of the waiting queue; on
    re-admission its prompt and what it had generated are run again as one prompt.  If the
    request in need is itself the newest, it is the one preempted;
  * a request that could not fit even into an empty cache, or is longer than
    ``max_model_len``, is finished at once with reason "unschedulable: ..."
    (atom/model_engine/scheduler.py:989-1050).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence as Seq

from ..cache import CacheManager, OutOfPages
from .sequence import Sequence, SequenceStatus


@dataclass
class ScheduledEntry:
    seq: Sequence
    start: int            # position of the first token of the portion
    num_tokens: int
    samples: bool         # the portion reaches the request's last token: a token is sampled


@dataclass
class ScheduledStep:
    entries: List[ScheduledEntry] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)
    rejected: List[Sequence] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.num_tokens for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 max_model_len: int, eos_token_ids: Seq[int] = (), portion_cap: int = 0,
                 enable_chunked_prefill: bool = True):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.eos_token_ids = tuple(eos_token_ids)
        self.portion_cap = portion_cap if portion_cap > 0 else max_num_batched_tokens
        self.enable_chunked_prefill = enable_chunked_prefill
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.num_preemptions = 0
        self.num_finished = 0

    # ------------------------------------------------------------------ queues

    def add(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def abort(self, seq_id: int, reason: str = "aborted") -> Optional[Sequence]:
        for q in (self.running, self.waiting):
            for s in list(q):
                if s.seq_id == seq_id:
                    q.remove(s)
                    if seq_id in self.cache.requests:
                        self.cache.release(seq_id)
                    self._finish(s, reason, release=False)
                    return s
        return None

    # ------------------------------------------------------------------ one step

    def _unschedulable_reason(self, seq: Sequence) -> Optional[str]:
        if seq.num_tokens > self.max_model_len:
            return f"unschedulable: {seq.num_tokens} tokens exceed max_model_len {self.max_model_len}"
        if not self.cache.fits_at_all(seq.num_tokens + 1, self.portion_cap):
            return "unschedulable: the request needs more cache pages than the pool has"
        if not self.enable_chunked_prefill and seq.num_tokens > self.max_num_batched_tokens:
            return "unschedulable: the prompt exceeds max_num_batched_tokens and portions are off"
        return None

    def _preempt(self, seq: Sequence, step: ScheduledStep) -> None:
        self.running.remove(seq)
        self.cache.release(seq.seq_id)
        seq.status = SequenceStatus.WAITING
        seq.num_computed = 0
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)
        step.preempted.append(seq)
        step.entries = [e for e in step.entries if e.seq is not seq]

    def _make_room(self, seq: Sequence, target: int, step: ScheduledStep) -> bool:
        """Takes pages for positions [0, target) of a running request, preempting newer
        requests while it must.  False: the request itself was preempted."""
        while True:
            try:
                self.cache.extend(seq.seq_id, target)
                return True
            except OutOfPages:
                victim = self.running[-1]
                self._preempt(victim, step)
                if victim is seq:
                    return False

    def schedule(self) -> ScheduledStep:
        step = ScheduledStep()
        budget = self.max_num_batched_tokens

        # 1. decoding requests and 2. requests inside their prompt, oldest first
        for phase in ("decode", "prompt"):
            for seq in list(self.running):
                if seq not in self.running or budget <= 0:
                    continue
                left = seq.num_uncomputed
                if (phase == "decode") != (left == 1):
                    continue
                n = min(left, self.portion_cap, budget)
                if not self.enable_chunked_prefill and n < left:
                    continue
                if not self._make_room(seq, seq.num_computed + n, step):
                    continue
                step.entries.append(ScheduledEntry(seq, seq.num_computed, n, seq.num_computed + n == seq.num_tokens))
                budget -= n

        # 3. admissions, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            why = self._unschedulable_reason(seq)
            if why is not None:
                self.waiting.popleft()
                self._finish(seq, why, release=False)
                step.rejected.append(seq)
                continue
            if seq in step.preempted:
                break  # preempted in this very step: it comes back in a later one
            if not self.cache.can_admit(seq.num_tokens + 1, self.portion_cap):
                break
            self.cache.admit(seq.seq_id)
            hit = self.cache.claim_prefix(seq.seq_id, seq.token_ids)   # tokens whose pages an earlier request left
            n = min(seq.num_tokens - hit, self.portion_cap, budget)
            if not self.enable_chunked_prefill and hit + n < seq.num_tokens:
                self.cache.release(seq.seq_id)
                break
            self.waiting.popleft()
            self.cache.extend(seq.seq_id, hit + n)
            seq.status = SequenceStatus.RUNNING
            seq.num_computed = hit
            self.running.append(seq)
            step.entries.append(ScheduledEntry(seq, hit, n, hit + n == seq.num_tokens))
            budget -= n
        return step

    # ------------------------------------------------------------------ after the step

    def _finish(self, seq: Sequence, reason: str, release: bool = True) -> None:
        seq.status = SequenceStatus.FINISHED
        seq.finish_reason = reason
        seq.finish_time = time.perf_counter()
        self.num_finished += 1
        if release and seq.seq_id in self.cache.requests:
            self.cache.release(seq.seq_id)

    def postprocess(self, step: ScheduledStep, sampled: Seq[int],
                    logprobs: Optional[Seq[float]] = None) -> List[Sequence]:
        """``sampled``: one token for every entry with ``samples`` set, in order (``logprobs``: their
        log-probabilities, if some request asked for them).  Advances the requests, appends tokens,
        applies the stop rules in the reference's order: stop sequences, EOS unless ignore_eos,
        stop_token_ids, max_tokens (atom/model_engine/scheduler.py:2298-2329)."""
        finished = []
        it = iter(sampled)
        lp = iter(logprobs) if logprobs is not None else None
        for e in step.entries:
            seq = e.seq
            if seq.is_finished:      # ended while this (look-ahead) step was in flight: its token is dropped
                if e.samples:
                    next(it, None)
                    if lp is not None:
                        next(lp, None)
                continue
            seq.num_computed = e.start + e.num_tokens
            if not e.samples:
                self.cache.publish(seq.seq_id, seq.token_ids)
                continue
            tok = int(next(it))
            seq.append_token(tok)
            self.cache.publish(seq.seq_id, seq.token_ids)     # (before a finished request's pages are let go)
            if lp is not None:
                v = float(next(lp))
                if seq.return_logprobs:
                    seq.logprobs.append(v)
            reason = None
            if any(len(st) <= seq.num_tokens and seq.token_ids[-len(st):] == st for st in seq.stop_token_sequences):
                reason = "stop_sequence"
            elif not seq.params.ignore_eos and tok in self.eos_token_ids:
                reason = "eos"
            elif tok in seq.params.stop_token_ids:
                reason = f"stop_{tok}"
            elif seq.num_output_tokens >= seq.params.max_tokens:
                reason = "max_tokens"
            elif seq.num_tokens >= self.max_model_len:
                reason = "max_model_len"
            if reason is not None:
                self.running.remove(seq)
                self._finish(seq, reason)
                finished.append(seq)
        return finished
