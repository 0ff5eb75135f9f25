"""One step's batch: the tokens each request brings, flattened, with the small integer
arrays the kernels read (positions, owning request, block tables, rows whose logits are
wanted).  Prompt portions and single decoded tokens lie side by side; a decoded token is
simply a portion of length one.  Replaces the reference's ScheduledBatch plus attention
metadata (atom/model_engine/scheduler.py:331-568, atom/model_ops/attentions/backends.py:374-497)
with one structure that is passed explicitly.

``StepBuilder`` packs those arrays into pinned host memory and brings them to the device in
one copy.  With a fixed shape (``build_fixed``) the arrays always lie at the same device
addresses and have the same sizes, whatever the number of live requests: rows beyond the
live ones are padding (``seq_of_token = -1``, no tokens, context length 0) that every kernel
skips.  That is the form a captured CUDA graph replays.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import NO_PAGE, CacheManager


class StepError(RuntimeError):
    pass


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
    seq_of_token: torch.Tensor         # [T] int32, row of the block tables (-1: padding row)
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
    # True while a step of a fixed shape is recorded into a graph that later steps of other makeups
    # replay: launch plans must then hold for every batch of num_tokens tokens in num_seqs requests
    # (the host lists above describe no particular batch)
    plan_for_any_batch: bool = False


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


class _Staging:
    """A device buffer with a ring of pinned host mirrors: a mirror is written again only
    after the copy that read it has finished."""

    def __init__(self, n: int, device, ring: int = 4):
        self.n = n
        self.dev = torch.zeros(n, dtype=torch.int32, device=device)
        self.host = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(ring)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * ring
        self.next = 0

    def acquire(self):
        k = self.next
        self.next = (k + 1) % len(self.host)
        if self.events[k] is not None:
            self.events[k].synchronize()
        return k, self.host[k].numpy()

    def push(self, k: int, total: int) -> None:
        self.dev[:total].copy_(self.host[k][:total], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[k] = ev


class StepBuilder:
    def __init__(self, cache: CacheManager, device, vocab_size: int, status: torch.Tensor):
        self.cache = cache
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.status = status
        self._flex = _Staging(1 << 16, self.device)
        self._fixed: Dict[object, _Staging] = {}     # batch size, or (tokens, requests), -> arrays of that shape
        self.h2d_bytes = 0

    # ------------------------------------------------------------------ shared

    def _fill(self, host, layout, entries, targets, S_pad: int, T_pad: int, widths):
        cache = self.cache
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        q_starts = [t - n for t, n in zip(targets, q_lens)]
        T = sum(q_lens)
        cu = np.zeros(S_pad + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu[1:S + 1])
        cu[S + 1:] = T
        rows: List[int] = []
        for i, e in enumerate(entries):
            for w in e.want:
                if not 0 <= w < q_lens[i]:
                    raise StepError(f"request {e.rid!r}: wanted place {w} outside its {q_lens[i]} tokens")
                rows.append(int(cu[i]) + int(w))

        def sec(name):
            o, n = layout[name]
            return host[o:o + n]

        tok, pos, sot = sec("token_ids"), sec("positions"), sec("seq_of_token")
        for i, e in enumerate(entries):
            a, b = cu[i], cu[i + 1]
            tok[a:b] = np.asarray(e.tokens, dtype=np.int64)
            pos[a:b] = np.arange(q_starts[i], targets[i], dtype=np.int32)
            sot[a:b] = i
        if T and (tok[:T].min() < 0 or tok[:T].max() >= self.vocab_size):
            raise StepError(f"token id outside [0, {self.vocab_size})")
        tok[T:T_pad] = 0
        pos[T:T_pad] = 0
        sot[T:T_pad] = -1
        sec("cu_q")[:] = cu
        cl = sec("ctx_len")
        cl[:S] = targets
        cl[S:] = 0
        slots = [cache.requests[e.rid].state_slot for e in entries]
        ss = sec("state_slots")
        ss[:S] = slots
        ss[S:] = 0
        for g, w in zip(cache.groups, widths):
            bt = sec(f"bt{g.index}").reshape(S_pad, w)
            bt[:] = NO_PAGE
            for i, e in enumerate(entries):
                t = cache.table(e.rid, g.index)
                bt[i, :len(t)] = t
        return q_lens, q_starts, slots, rows

    def _context(self, dev, layout, T, S, R, widths, q_lens, q_starts, slots, targets) -> StepContext:
        def dsec(name):
            o, n = layout[name]
            return dev[o:o + n]

        return StepContext(
            num_tokens=T, num_seqs=S, num_logits_rows=R,
            token_ids=dsec("token_ids"), positions=dsec("positions"), seq_of_token=dsec("seq_of_token"),
            cu_q=dsec("cu_q"), ctx_len=dsec("ctx_len"), state_slots=dsec("state_slots"),
            logits_rows=dsec("logits_rows")[:R],
            block_tables={g.index: dsec(f"bt{g.index}").view(S, w) for g, w in zip(self.cache.groups, widths)},
            status=self.status, q_lens=q_lens, q_starts=q_starts, host_state_slots=slots,
            max_q_len=max(q_lens, default=0), max_ctx_len=max(targets, default=0),
        )

    # ------------------------------------------------------------------ any shape

    def build(self, entries: Sequence[StepEntry], targets: List[int]) -> StepContext:
        """Arrays sized for exactly this batch.  ``targets[i]``: tokens of request i in the
        cache after the step."""
        cache = self.cache
        S = len(entries)
        T = sum(len(e.tokens) for e in entries)
        R = sum(len(e.want) for e in entries)
        widths = [max(1, max(len(cache.table(e.rid, g.index)) for e in entries)) for g in cache.groups]
        layout, total = pack_layout(T, S, R, widths)
        if total > self._flex.n:
            self._flex = _Staging(1 << (total - 1).bit_length(), self.device)
        k, host = self._flex.acquire()
        q_lens, q_starts, slots, rows = self._fill(host, layout, entries, targets, S, T, widths)
        o, n = layout["logits_rows"]
        host[o:o + n] = 0
        host[o:o + R] = rows
        self._flex.push(k, total)
        self.h2d_bytes += 4 * total
        return self._context(self._flex.dev, layout, T, S, R, widths, q_lens, q_starts, slots, targets)

    # ------------------------------------------------------------------ fixed shape

    def fixed_layout(self, batch: int, table_width: int):
        widths = [table_width] * len(self.cache.groups)
        return pack_layout(batch, batch, batch, widths), widths

    def build_fixed(self, entries: Sequence[StepEntry], targets: List[int], batch: int,
                    table_width: int, token_rows: Optional[Sequence[int]] = None) -> StepContext:
        """Arrays of a fixed shape for ``batch`` single-token requests (the live ones first,
        padding after them), always at the same device addresses for this ``batch``.  The
        logits of all ``batch`` rows are computed; the caller picks the wanted ones.

        token_rows: the token section carries these numbers instead of the entries' tokens
        (the caller then replaces them on the device by tokens it gathers with them)."""
        assert len(entries) <= batch and all(len(e.tokens) == 1 for e in entries)
        (layout, total), widths = self.fixed_layout(batch, table_width)
        st = self._fixed.get(batch)
        if st is None:
            st = self._fixed[batch] = _Staging(total, self.device)
        k, host = st.acquire()
        q_lens, q_starts, slots, _ = self._fill(host, layout, entries, targets, batch, batch, widths)
        o, n = layout["logits_rows"]
        host[o:o + n] = np.arange(batch, dtype=np.int32)
        if token_rows is not None:
            o, _ = layout["token_ids"]
            host[o:o + len(entries)] = np.asarray(token_rows, dtype=np.int32)
        st.push(k, total)
        self.h2d_bytes += 4 * total
        ctx = self._context(st.dev, layout, batch, batch, batch, widths, q_lens, q_starts, slots, targets)
        # host lists describe the padded batch: padding requests bring one skipped row each
        ctx.q_lens = q_lens + [1] * (batch - len(entries))
        return ctx

    # ------------------------------------------------------------------ fixed shape, any makeup

    def build_fixed_mixed(self, entries: Sequence[StepEntry], targets: List[int], tokens: int, seqs: int,
                          table_width: int) -> StepContext:
        """Arrays of a fixed shape for up to ``tokens`` tokens of up to ``seqs`` requests with up to
        ``seqs`` wanted rows, portions and single tokens alike, always at the same device addresses
        for this pair of sizes; what is beyond the live tokens and requests is padding."""
        S, T = len(entries), sum(len(e.tokens) for e in entries)
        assert S <= seqs and T <= tokens
        widths = [table_width] * len(self.cache.groups)
        layout, total = pack_layout(tokens, seqs, seqs, widths)
        key = (tokens, seqs)
        st = self._fixed.get(key)
        if st is None:
            st = self._fixed[key] = _Staging(total, self.device)
        k, host = st.acquire()
        q_lens, q_starts, slots, rows = self._fill(host, layout, entries, targets, seqs, tokens, widths)
        if len(rows) > seqs:
            raise StepError(f"{len(rows)} wanted rows in a step shaped for {seqs}")
        o, n = layout["logits_rows"]
        host[o:o + n] = 0
        host[o:o + len(rows)] = rows
        st.push(k, total)
        self.h2d_bytes += 4 * total
        ctx = self._context(st.dev, layout, tokens, seqs, seqs, widths, q_lens, q_starts, slots, targets)
        ctx.q_lens = q_lens + [0] * (seqs - S)
        return ctx

    def fixed_context_mixed(self, tokens: int, seqs: int, table_width: int, max_ctx_len: int) -> StepContext:
        """The context over the fixed-shape arrays of (tokens, seqs) without touching them, for a graph
        capture.  ``build_fixed_mixed`` must have run once for this pair."""
        widths = [table_width] * len(self.cache.groups)
        layout, _ = pack_layout(tokens, seqs, seqs, widths)
        st = self._fixed[(tokens, seqs)]
        ctx = self._context(st.dev, layout, tokens, seqs, seqs, widths, [tokens] + [0] * (seqs - 1), [0] * seqs,
                            [0] * seqs, [max_ctx_len] * seqs)
        ctx.plan_for_any_batch = True
        return ctx

    def fixed_context(self, batch: int, table_width: int, max_ctx_len: int) -> StepContext:
        """The context over the fixed-shape arrays of ``batch`` without touching them: what a
        graph capture records its launches against.  ``build_fixed`` must have run once."""
        (layout, _), widths = self.fixed_layout(batch, table_width)
        st = self._fixed[batch]
        ctx = self._context(st.dev, layout, batch, batch, batch, widths, [1] * batch, [0] * batch,
                            [0] * batch, [max_ctx_len] * batch)
        return ctx
