"""Builders of replay traces: the same requests cut into steps in different ways.

A trace is a list of steps {"step", "entries": [{"id", "tokens", "want"}], "end"} in the
format ``bin/trace_run`` reads.  Every builder asks for the logits at every position, so
that all cuts can be compared position by position."""
from __future__ import annotations

from typing import Dict, List, Sequence


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def whole(seqs: Dict[str, Sequence[int]]) -> List[dict]:
    """Each request alone, whole, in one step."""
    steps = []
    for rid, toks in seqs.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def tail_by_token(seqs: Dict[str, Sequence[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in seqs.items():
        toks = list(toks)
        head = max(1, len(toks) - tail) if len(toks) > tail else 1
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def ragged(seqs: Dict[str, Sequence[int]], sizes: Sequence[int] = (13, 5, 2, 29, 2, 8, 3, 17)) -> List[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    k = 0
    for rid, toks in seqs.items():
        toks = list(toks)
        i = 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}], "end": []})
            i += n
        steps[-1]["end"] = [rid]
    return steps


def mixed(seqs: Dict[str, Sequence[int]], max_live: int = 4, tail: int = 12,
          sizes: Sequence[int] = (7, 2, 19, 4, 11, 2, 30), budget_tokens: int = 0, page: int = 64):
    """Up to ``max_live`` requests at a time: portions of some beside single decoded tokens
    of others.  A request enters when a place is free and, if ``budget_tokens`` is set, when
    the live requests' final lengths (rounded up to ``page``) leave room for it, so that the
    pool is small and pages are used again.  Returns (steps, most tokens held at a time)."""
    waiting = [(rid, list(t)) for rid, t in seqs.items()]
    live: List[dict] = []
    steps, peak, k = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting[0]
            held = sum(_round_up(len(r["toks"]), page) for r in live)
            if budget_tokens and live and held + _round_up(len(toks), page) > budget_tokens:
                break
            waiting.pop(0)
            live.append({"rid": rid, "toks": toks, "done": 0})
        peak = max(peak, sum(_round_up(len(r["toks"]), page) for r in live))
        entries, ended = [], []
        for j, r in enumerate(live):
            left = len(r["toks"]) - r["done"]
            if left <= tail:
                n = 1                                   # decoding: one token a step
            else:
                n = min(sizes[k % len(sizes)], left - tail)
                k += 1
            # a request may sit out a step and go on later
            if (len(steps) + j) % 5 == 4 and len(live) > 1:
                continue
            entries.append({"id": r["rid"], "tokens": r["toks"][r["done"]:r["done"] + n], "want": list(range(n))})
            r["done"] += n
            if r["done"] == len(r["toks"]):
                ended.append(r["rid"])
        live = [r for r in live if r["done"] < len(r["toks"])]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps, peak


def mixed_refeed(seqs: Dict[str, Sequence[int]], victims: Sequence[str], **kw):
    """The mixed trace in which each request named in ``victims`` is ended about half-way (its pages go
    back while the others go on) and fed again from its first token under the same id: what a scheduler
    does when it preempts a request and computes it again (atom/model_engine/scheduler.py:1928-1952).
    Entries carry "pos", the position of their first token, so that ``collect_rows`` can tell the two
    passes apart.  Returns (steps, most tokens held at a time)."""
    max_live, tail = kw.get("max_live", 4), kw.get("tail", 12)
    sizes, budget_tokens, page = kw.get("sizes", (7, 2, 19, 4, 11, 2, 30)), kw.get("budget_tokens", 0), kw.get("page", 64)
    waiting = [(rid, list(t)) for rid, t in seqs.items()]
    live: List[dict] = []
    todo = set(victims)
    steps, peak, k = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting[0]
            held = sum(_round_up(len(r["toks"]), page) for r in live)
            if budget_tokens and live and held + _round_up(len(toks), page) > budget_tokens:
                break
            waiting.pop(0)
            live.append({"rid": rid, "toks": toks, "done": 0})
        peak = max(peak, sum(_round_up(len(r["toks"]), page) for r in live))
        entries, ended = [], []
        for j, r in enumerate(live):
            left = len(r["toks"]) - r["done"]
            if left <= tail:
                n = 1
            else:
                n = min(sizes[k % len(sizes)], left - tail)
                k += 1
            if (len(steps) + j) % 5 == 4 and len(live) > 1:
                continue
            entries.append({"id": r["rid"], "tokens": r["toks"][r["done"]:r["done"] + n], "want": list(range(n)),
                            "pos": r["done"]})
            r["done"] += n
            if r["done"] == len(r["toks"]):
                ended.append(r["rid"])
            elif r["rid"] in todo and r["done"] >= len(r["toks"]) // 2:
                todo.discard(r["rid"])       # preempted: everything it holds goes back; it starts over
                ended.append(r["rid"])
                r["done"] = 0
        live = [r for r in live if r["done"] < len(r["toks"]) or r["rid"] in ended and r["done"] == 0]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    assert not todo, f"never preempted: {sorted(todo)}"
    return steps, peak


def collect_rows(steps: List[dict], outputs: Dict[int, "object"]):
    """{request: [(position, logits row), ...]} in the order computed; a request that was fed twice
    has its early positions twice."""
    per: Dict[str, List] = {}
    for s in steps:
        arr = outputs.get(s["step"])
        r = 0
        for e in s["entries"]:
            for w in e["want"]:
                per.setdefault(e["id"], []).append((e["pos"] + w, arr[r]))
                r += 1
    return per


def collect(steps: List[dict], outputs: Dict[int, "object"]):
    """Maps the per-step logits back to {request: [per-position logits rows]}."""
    import numpy as np

    per: Dict[str, List] = {}
    for s in steps:
        arr = outputs.get(s["step"])
        r = 0
        for e in s["entries"]:
            for _ in e["want"]:
                per.setdefault(e["id"], []).append(arr[r])
                r += 1
    return {k: np.stack(v) for k, v in per.items()}
