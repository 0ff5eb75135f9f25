"""Device arrays behind the cache manager's accounting.

For every page group one array per entry that its mixers declare (CacheNeed.entries):
[slots, pages, *shape with the page's tokens before the last axis], e.g. keys and values of
(kv heads, head size) each as [slots, pages, kv heads, page size, head size].  And one array
[state slots, *shape] per cache slot whose mixer keeps fixed-size state, zero when a request is
admitted.  ``view(slot)`` is what a mixer gets for its run entry."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from .manager import CacheManager


@dataclass
class CacheView:
    slot: int
    group: int = -1                       # page group (index into StepContext.block_tables)
    page_size: int = 0
    pages: Dict[str, torch.Tensor] = field(default_factory=dict)   # entry name -> [pages, ..., page size, last]
    state: Optional[torch.Tensor] = None     # [state slots, *shape]

    @property
    def k_pages(self) -> Optional[torch.Tensor]:   # [pages, kv heads, page size, head size]
        return self.pages.get("k")

    @property
    def v_pages(self) -> Optional[torch.Tensor]:
        return self.pages.get("v")


def _entry_dtype(entry, compute: torch.dtype) -> torch.dtype:
    return compute if entry.dtype == "compute" else getattr(torch, entry.dtype)


def _page_shape(entry, page_size: int):
    return tuple(entry.shape[:-1]) + (page_size, entry.shape[-1])


class CacheStorage:
    def __init__(self, manager: CacheManager, dtype: torch.dtype, device):
        self.manager = manager
        self.arrays = []
        self._views: Dict[int, CacheView] = {}
        self._states = []
        ps = manager.page_size
        for g in manager.groups:
            per_entry = {}
            for e in g.entries:
                a = torch.zeros((len(g.slots), g.pool.num_pages) + _page_shape(e, ps),
                                dtype=_entry_dtype(e, dtype), device=device)
                self.arrays.append(a)
                per_entry[e.name] = a
            for i, slot in enumerate(g.slots):
                self._views[slot] = CacheView(slot, g.index, ps, {n: a[i] for n, a in per_entry.items()})
        for slot, need in manager.state_needs.items():
            sdt = dtype if need.state_dtype == "compute" else getattr(torch, need.state_dtype)
            st = torch.zeros((manager.state_slots.num_slots,) + tuple(need.state_shape), dtype=sdt, device=device)
            self.arrays.append(st)
            self._states.append(st)
            self._views[slot] = CacheView(slot, state=st)
        if self._states:
            manager.admit_hooks.append(self.clear_state)

    def clear_state(self, state_slot: int) -> None:
        """Zeroes a request slot's rows in every state array.  Runs when a request is admitted (a
        preempted request that comes back included), so a mixer finds zeros at a request's first
        token whoever held the slot before."""
        for st in self._states:
            st[state_slot].zero_()

    def view(self, slot: int) -> Optional[CacheView]:
        return self._views.get(slot)

    def get(self, slot: int) -> Optional[CacheView]:   # mapping-style access used by Model.forward
        return self._views.get(slot)

    def bytes(self) -> int:
        return sum(a.numel() * a.element_size() for a in self.arrays)

    @staticmethod
    def bytes_per_page(manager: CacheManager, dtype: torch.dtype) -> int:
        """Bytes that one more page in every group costs."""
        total = 0
        for g in manager.groups:
            for e in g.entries:
                n = manager.page_size
                for d in e.shape:
                    n *= d
                total += len(g.slots) * n * torch.empty((), dtype=_entry_dtype(e, dtype)).element_size()
        return total
