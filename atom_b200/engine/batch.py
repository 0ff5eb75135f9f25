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
skips.  That is the form a captured CUDA graph replays.  Its block tables have rows as long as the
longest request the engine takes, but a step fills and copies only the live requests' rows as far
as their longest context reaches, so a step's host work and copy do not grow with ``max_model_len``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import native
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


class _HostRing:
    """A ring of pinned host buffers that steps fill and copy from: a buffer is written again only
    after the copies that read it have finished.  One ring serves steps of every shape (they run one
    after another)."""

    def __init__(self, ring: int = 4):
        self.host: List[Optional[torch.Tensor]] = [None] * ring
        self.events: List[Optional[torch.cuda.Event]] = [None] * ring
        self.next = 0

    def acquire(self, n: int):
        """(slot, pinned tensor of at least n int32, its numpy view)."""
        k = self.next
        self.next = (k + 1) % len(self.host)
        if self.events[k] is not None:
            self.events[k].synchronize()
        buf = self.host[k]
        if buf is None or buf.numel() < n:
            buf = self.host[k] = torch.zeros(max(1 << 14, 1 << (n - 1).bit_length()), dtype=torch.int32).pin_memory()
        return k, buf, buf.numpy()

    def sent(self, k: int) -> None:
        """The copies out of slot k have been put on the stream."""
        ev = torch.cuda.Event()
        ev.record()
        self.events[k] = ev


class _FixedArrays:
    """Device arrays of one fixed shape: the small per-token and per-request arrays, then one block
    table per page group, ``width`` entries a row.  They keep their addresses for good (a captured
    graph reads them); a step overwrites the small arrays and, of the tables, the rows of its live
    requests as far as their longest context reaches.  What lies beyond is left over from earlier
    steps and never read: a kernel looks up only pages below a request's context length."""

    def __init__(self, tokens: int, seqs: int, num_groups: int, width: int, device):
        self.tokens, self.seqs, self.width = tokens, seqs, width
        self.layout, total = pack_layout(tokens, seqs, seqs, [width] * num_groups)
        self.small = self.layout["bt0"][0] if num_groups else total      # int32 elements before the tables
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)


class StepBuilder:
    def __init__(self, cache: CacheManager, device, vocab_size: int, status: torch.Tensor):
        self.cache = cache
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.status = status
        self._ring = _HostRing()
        self._flex_dev = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        self._fixed: Dict[object, _FixedArrays] = {}     # batch size, or (tokens, requests), -> arrays of that shape
        self.h2d_bytes = 0

    # ------------------------------------------------------------------ shared

    def _fill(self, host, layout, entries, targets, S_pad: int, T_pad: int, widths):
        """Writes the step's arrays into ``host`` after ``layout``; tables are S_pad rows of widths[g]."""
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
            o, n = layout[f"bt{g.index}"]
            bt = host[o:o + n].reshape(-1, w)
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

    def _live_widths(self, entries) -> List[int]:
        cache = self.cache
        return [max(1, max((len(cache.table(e.rid, g.index)) for e in entries), default=1)) for g in cache.groups]

    # ------------------------------------------------------------------ any shape

    def build(self, entries: Sequence[StepEntry], targets: List[int]) -> StepContext:
        """Arrays sized for exactly this batch.  ``targets[i]``: tokens of request i in the
        cache after the step."""
        S = len(entries)
        T = sum(len(e.tokens) for e in entries)
        R = sum(len(e.want) for e in entries)
        widths = self._live_widths(entries)
        layout, total = pack_layout(T, S, R, widths)
        if total > self._flex_dev.numel():
            self._flex_dev = torch.zeros(1 << (total - 1).bit_length(), dtype=torch.int32, device=self.device)
        k, pinned, host = self._ring.acquire(total)
        q_lens, q_starts, slots, rows = self._fill(host, layout, entries, targets, S, T, widths)
        o, n = layout["logits_rows"]
        host[o:o + n] = 0
        host[o:o + R] = rows
        self._flex_dev[:total].copy_(pinned[:total], non_blocking=True)
        self._ring.sent(k)
        self.h2d_bytes += 4 * total
        return self._context(self._flex_dev, layout, T, S, R, widths, q_lens, q_starts, slots, targets)

    # ------------------------------------------------------------------ fixed shape

    def _arrays(self, key, tokens: int, seqs: int, table_width: int) -> _FixedArrays:
        fa = self._fixed.get(key)
        if fa is None:
            fa = self._fixed[key] = _FixedArrays(tokens, seqs, len(self.cache.groups), table_width, self.device)
        assert fa.width == table_width
        return fa

    def _send_fixed(self, fa: _FixedArrays, entries, targets, token_rows=None, all_rows=False):
        """Fills a host buffer with the step's small arrays (in the device layout) and, behind them, its
        tables cut down to the live requests and their longest context; two kinds of copies bring them
        to their places: one for the small arrays, one of rows for each table."""
        S = len(entries)
        live = self._live_widths(entries) if S else []
        # host layout: the device's small arrays, then compact tables [S, live width]
        layout = dict(fa.layout)
        cur = fa.small
        for g, w in zip(self.cache.groups, live):
            layout[f"bt{g.index}"] = (cur, S * w)
            cur += S * w
        k, pinned, host = self._ring.acquire(cur)
        q_lens, q_starts, slots, rows = self._fill(host, layout, entries, targets, fa.seqs, fa.tokens, live)
        o, n = layout["logits_rows"]
        if all_rows:
            host[o:o + n] = np.arange(n, dtype=np.int32)
        else:
            if len(rows) > fa.seqs:
                raise StepError(f"{len(rows)} wanted rows in a step shaped for {fa.seqs}")
            host[o:o + n] = 0
            host[o:o + len(rows)] = rows
        if token_rows is not None:
            o, _ = layout["token_ids"]
            host[o:o + S] = np.asarray(token_rows, dtype=np.int32)
        fa.dev[:fa.small].copy_(pinned[:fa.small], non_blocking=True)
        sent = fa.small
        for g, w in zip(self.cache.groups, live):
            o, n = layout[f"bt{g.index}"]
            do, _ = fa.layout[f"bt{g.index}"]
            native.copy_rows_h2d(fa.dev[do:], fa.width, pinned[o:], w, w, S)
            sent += n
        self._ring.sent(k)
        self.h2d_bytes += 4 * sent
        return q_lens, q_starts, slots

    def build_fixed(self, entries: Sequence[StepEntry], targets: List[int], batch: int,
                    table_width: int, token_rows: Optional[Sequence[int]] = None) -> StepContext:
        """Arrays of a fixed shape for ``batch`` single-token requests (the live ones first,
        padding after them), always at the same device addresses for this ``batch``.  The
        logits of all ``batch`` rows are computed; the caller picks the wanted ones.

        token_rows: the token section carries these numbers instead of the entries' tokens
        (the caller then replaces them on the device by tokens it gathers with them)."""
        assert len(entries) <= batch and all(len(e.tokens) == 1 for e in entries)
        fa = self._arrays(batch, batch, batch, table_width)
        q_lens, q_starts, slots = self._send_fixed(fa, entries, targets, token_rows, all_rows=True)
        widths = [table_width] * len(self.cache.groups)
        ctx = self._context(fa.dev, fa.layout, batch, batch, batch, widths, q_lens, q_starts, slots, targets)
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
        fa = self._arrays((tokens, seqs), tokens, seqs, table_width)
        q_lens, q_starts, slots = self._send_fixed(fa, entries, targets)
        widths = [table_width] * len(self.cache.groups)
        ctx = self._context(fa.dev, fa.layout, tokens, seqs, seqs, widths, q_lens, q_starts, slots, targets)
        ctx.q_lens = q_lens + [0] * (seqs - S)
        return ctx

    def fixed_context_mixed(self, tokens: int, seqs: int, table_width: int, max_ctx_len: int) -> StepContext:
        """The context over the fixed-shape arrays of (tokens, seqs) without touching them, for a graph
        capture; launch plans are made for requests of up to ``max_ctx_len`` tokens."""
        fa = self._arrays((tokens, seqs), tokens, seqs, table_width)
        widths = [table_width] * len(self.cache.groups)
        ctx = self._context(fa.dev, fa.layout, tokens, seqs, seqs, widths, [tokens] + [0] * (seqs - 1), [0] * seqs,
                            [0] * seqs, [max_ctx_len] * seqs)
        ctx.plan_for_any_batch = True
        return ctx

    def fixed_context(self, batch: int, table_width: int, max_ctx_len: int) -> StepContext:
        """The context over the fixed-shape arrays of ``batch`` without touching them: what a
        graph capture records its launches against; launch plans are made for requests of up to
        ``max_ctx_len`` tokens."""
        fa = self._arrays(batch, batch, batch, table_width)
        widths = [table_width] * len(self.cache.groups)
        return self._context(fa.dev, fa.layout, batch, batch, batch, widths, [1] * batch, [0] * batch,
                             [0] * batch, [max_ctx_len] * batch)
