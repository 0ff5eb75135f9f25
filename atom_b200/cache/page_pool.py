"""A pool of fixed-size cache pages: hands out the lowest free ids first (so that runs are
reproducible and freed pages are used again at once), knows who holds every page, and
refuses to free a page twice.  After the reference's BlockPool (vacant min-heap,
atom/model_engine/block_pool.py:26-60,175-219) without its prefix-cache half."""
from __future__ import annotations

import heapq
from typing import Dict, Hashable, Iterable, List, Optional


class OutOfPages(RuntimeError):
    """The pool cannot give as many pages as were asked for; nothing was taken."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages))
        heapq.heapify(self._free)
        self._owner: Dict[int, Hashable] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return len(self._owner)

    def allocate(self, n: int, owner: Hashable) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"asked for {n} pages, {len(self._free)} free of {self.num_pages}")
        out = [heapq.heappop(self._free) for _ in range(n)]
        for p in out:
            self._owner[p] = owner
        return out

    def free(self, pages: Iterable[int], owner: Optional[Hashable] = None) -> None:
        pages = list(pages)
        for p in pages:
            if p not in self._owner:
                raise RuntimeError(f"page {p} freed twice or never allocated")
            if owner is not None and self._owner[p] != owner:
                raise RuntimeError(f"page {p} is held by {self._owner[p]!r}, freed by {owner!r}")
        if len(set(pages)) != len(pages):
            raise RuntimeError("a page is named twice in one free")
        for p in pages:
            del self._owner[p]
            heapq.heappush(self._free, p)

    def owner_of(self, page: int) -> Optional[Hashable]:
        return self._owner.get(page)

    def check(self) -> None:
        """Every page is either free or held, never both, never twice, none lost."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise AssertionError("a page is in the free list twice")
        if set(free) & set(self._owner):
            raise AssertionError("a page is both free and held")
        if len(free) + len(self._owner) != self.num_pages:
            raise AssertionError(
                f"pages lost: {len(free)} free + {len(self._owner)} held != {self.num_pages}"
            )
