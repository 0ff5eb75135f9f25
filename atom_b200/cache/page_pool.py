"""A pool of fixed-size cache pages: hands out the lowest free ids first (so that runs are
reproducible and freed pages are used again at once), knows who holds every page, and
refuses to free a page twice.  After the reference's BlockPool (vacant min-heap plus an LRU
of cached pages, atom/model_engine/block_pool.py:26-60,153-219).

With prefix caching a page may be held by several requests at once (``share``), and a page
whose content has been published under a key stays findable after its last holder has let
go of it: it then waits in an LRU of cached pages, counts as free, and is taken (and its key
forgotten) only when the vacant pages do not suffice: handing a page out is the eviction.
"""
from __future__ import annotations

import heapq
from collections import OrderedDict
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
        self._holders: Dict[int, List[Hashable]] = {}      # page -> who holds it (one entry without sharing)
        self._cached: "OrderedDict[int, Hashable]" = OrderedDict()   # held by nobody, content published: page -> key
        self._key_of: Dict[int, Hashable] = {}
        self._page_of: Dict[Hashable, int] = {}
        self.num_evictions = 0

    @property
    def num_free(self) -> int:
        return len(self._free) + len(self._cached)

    @property
    def num_used(self) -> int:
        return len(self._holders)

    @property
    def num_cached(self) -> int:
        return len(self._cached)

    def allocate(self, n: int, owner: Hashable) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > self.num_free:
            raise OutOfPages(f"asked for {n} pages, {self.num_free} free of {self.num_pages}")
        out = []
        for _ in range(n):
            if self._free:
                p = heapq.heappop(self._free)
            else:                      # the least recently released cached page: its content is given up
                p, key = self._cached.popitem(last=False)
                del self._key_of[p]
                del self._page_of[key]
                self.num_evictions += 1
            self._holders[p] = [owner]
            out.append(p)
        return out

    def free(self, pages: Iterable[int], owner: Optional[Hashable] = None) -> None:
        """``owner`` lets go of the pages.  A page nobody holds any more becomes vacant, or, if its
        content is published, cached (most recently released last)."""
        pages = list(pages)
        for p in pages:
            if p not in self._holders:
                raise RuntimeError(f"page {p} freed twice or never allocated")
            if owner is not None and owner not in self._holders[p]:
                raise RuntimeError(f"page {p} is held by {self._holders[p]!r}, freed by {owner!r}")
        if len(set(pages)) != len(pages):
            raise RuntimeError("a page is named twice in one free")
        for p in pages:
            holders = self._holders[p]
            holders.remove(owner if owner is not None else holders[0])
            if holders:
                continue
            del self._holders[p]
            key = self._key_of.get(p)
            if key is None:
                heapq.heappush(self._free, p)
            else:
                self._cached[p] = key

    # ------------------------------------------------------------------ sharing by content

    def lookup(self, key: Hashable) -> Optional[int]:
        """The page whose content was published under ``key``, held or cached; None if there is none."""
        return self._page_of.get(key)

    def share(self, page: int, owner: Hashable) -> None:
        """``owner`` takes a published page as one more holder (out of the cached ones if nobody held it)."""
        if page not in self._key_of:
            raise RuntimeError(f"page {page} is not published")
        if page in self._cached:
            del self._cached[page]
            self._holders[page] = [owner]
        else:
            if owner in self._holders[page]:
                raise RuntimeError(f"page {page} is already held by {owner!r}")
            self._holders[page].append(owner)

    def publish(self, page: int, key: Hashable) -> bool:
        """Makes a held page findable under ``key``.  False (and nothing changes) if another page
        already answers to the key or the page already has one."""
        if page not in self._holders:
            raise RuntimeError(f"page {page} is not held")
        if key in self._page_of or page in self._key_of:
            return False
        self._page_of[key] = page
        self._key_of[page] = key
        return True

    def key_of(self, page: int) -> Optional[Hashable]:
        return self._key_of.get(page)

    def owner_of(self, page: int) -> Optional[Hashable]:
        h = self._holders.get(page)
        return h[0] if h else None

    def holders_of(self, page: int) -> List[Hashable]:
        return list(self._holders.get(page, ()))

    def check(self) -> None:
        """Every page is vacant, cached or held, exactly one of them, none lost; keys and pages
        answer to each other."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise AssertionError("a page is in the free list twice")
        groups = (set(free), set(self._cached), set(self._holders))
        if groups[0] & groups[1] or groups[0] & groups[2] or groups[1] & groups[2]:
            raise AssertionError("a page is in two of: vacant, cached, held")
        if len(free) + len(self._cached) + len(self._holders) != self.num_pages:
            raise AssertionError(
                f"pages lost: {len(free)} vacant + {len(self._cached)} cached + {len(self._holders)} held "
                f"!= {self.num_pages}")
        for p, h in self._holders.items():
            if not h or len(set(h)) != len(h):
                raise AssertionError(f"page {p}: holders {h!r}")
        if len(self._key_of) != len(self._page_of) or any(self._page_of.get(k) != p for p, k in self._key_of.items()):
            raise AssertionError("keys and pages do not answer to each other")
        if any(self._key_of.get(p) != k for p, k in self._cached.items()):
            raise AssertionError("a cached page has lost its key")
        if any(p in groups[0] for p in self._key_of):
            raise AssertionError("a vacant page still has a key")
