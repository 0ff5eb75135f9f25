"""Slots for per-request state of fixed size (recurrent state, convolution tails, ...).

Every admitted request holds one slot id; mixers that declare a "state" cache need index
their per-slot arrays with it.  An architecture whose mixers keep no such state (Qwen3
dense) has zero arrays but the slot accounting is the same.  After the reference's
StateGroupPool (atom/model_engine/state_pool.py:107-172)."""
from __future__ import annotations

import heapq
from typing import Dict, Hashable, List


class OutOfSlots(RuntimeError):
    pass


class StateSlots:
    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("need at least one state slot")
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots))
        heapq.heapify(self._free)
        self._owner: Dict[int, Hashable] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, owner: Hashable) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} state slots are taken")
        s = heapq.heappop(self._free)
        self._owner[s] = owner
        return s

    def free(self, slot: int) -> None:
        if slot not in self._owner:
            raise RuntimeError(f"state slot {slot} freed twice or never allocated")
        del self._owner[slot]
        heapq.heappush(self._free, slot)

    def check(self) -> None:
        if len(set(self._free)) != len(self._free) or set(self._free) & set(self._owner):
            raise AssertionError("state slot accounting is inconsistent")
        if len(self._free) + len(self._owner) != self.num_slots:
            raise AssertionError("state slots lost")
