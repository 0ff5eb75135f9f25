"""Device arrays behind the cache manager's accounting.

One array per page group, [slots, 2 (keys, values), pages, kv heads, page size, head size]
in the compute type, and one array [state slots, *shape] per cache slot whose mixer keeps
fixed-size state, zero when a request is admitted.  ``view(slot)`` is what a mixer gets for its
run entry."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .manager import CacheManager


@dataclass
class CacheView:
    slot: int
    group: int = -1                       # page group (index into StepContext.block_tables)
    page_size: int = 0
    k_pages: Optional[torch.Tensor] = None   # [pages, kv heads, page size, head size]
    v_pages: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None     # [state slots, *shape]


class CacheStorage:
    def __init__(self, manager: CacheManager, dtype: torch.dtype, device):
        self.manager = manager
        self.arrays = []
        self._views: Dict[int, CacheView] = {}
        self._states = []
        ps = manager.page_size
        for g in manager.groups:
            a = torch.zeros(
                (len(g.slots), 2, g.pool.num_pages, g.num_kv_heads, ps, g.head_dim),
                dtype=dtype, device=device,
            )
            self.arrays.append(a)
            for i, slot in enumerate(g.slots):
                self._views[slot] = CacheView(slot, g.index, ps, a[i, 0], a[i, 1])
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
        es = torch.empty((), dtype=dtype).element_size()
        return sum(
            len(g.slots) * 2 * g.num_kv_heads * manager.page_size * g.head_dim * es for g in manager.groups
        )
