"""The cache manager: pages of keys and values with a block table per request, one page
pool per group of cache slots with the same need, and a state slot per request.

Cache slots (one per run-order entry that writes a cache) are grouped by what their mixer
keeps: (the arrays it holds per token, window).  A group has its own pool and its own block table
per request; all slots of a group share the table (page id p means page p of every slot's
storage in that group).  A group with a window gives pages back as soon as every position
on them is further back than any later query can look.

Accounting per request, in tokens:
  extend(id, n)   make room for positions [0, n): takes pages, may raise OutOfPages
  commit(id, n)   the step ran: n tokens are in the cache; pages a window has passed are freed
  release(id)     the request ended (or is preempted): everything goes back
After the reference's BlockManager (atom/model_engine/block_manager.py: can_allocate :371,
allocate :447, can_append :1109, may_append :1117, deallocate :1083), reshaped so that a
step may hold prompt portions and decoded tokens together.

Prefix caching (optional; the reference's chained block hashes, block_manager.py:181-187,
371-445, 558-666): a full page is published, once the step that filled it has run, under a
key that stands for all tokens from the request's first up to the page's last.  A new request
whose tokens begin the same way takes such pages as one more holder instead of computing
them (claim_prefix), all but its last token at most, so that there is always something to
compute.  Pages that nobody holds keep their content until the pool needs them (page_pool).
Only for models with one group of pages that keeps all keys and no per-request state.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Tuple

from ..parts.spec import CacheNeed
from .page_pool import OutOfPages, PagePool
from .state_slots import StateSlots

NO_PAGE = -1


@dataclass
class CacheGroup:
    index: int
    key: Tuple
    window: Optional[int]
    entries: Tuple                   # the CacheEntry arrays every slot of the group holds per token
    slots: List[int]                 # cache slots (run-order cache ids) stored in this group
    pool: PagePool = None            # type: ignore


@dataclass
class RequestCache:
    state_slot: int
    committed: int = 0               # tokens whose keys/values are in the cache
    reserved: int = 0                # positions [0, reserved) have pages (where still needed)
    tables: Dict[int, List[int]] = field(default_factory=dict)   # group -> page id per logical page
    published: int = 0               # leading pages that answer to a prefix key (claimed or published by this request)
    chain: Optional[int] = None      # key of the last of them


class CacheManager:
    def __init__(self, needs: Dict[int, CacheNeed], page_size: int, num_pages, max_requests: int,
                 prefix_caching: bool = False):
        """needs: cache slot -> CacheNeed.  num_pages: int (every group) or {group key: int}."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.prefix_caching = prefix_caching
        self._chains: Dict[Tuple, int] = {}      # (key of the pages before, the page's tokens) -> key
        self._chain_of: Dict[int, Tuple] = {}    # key -> that pair, to forget it when its page is given up
        self._next_key = 0
        self.prefix_hit_tokens = 0               # tokens that requests did not have to compute
        self.prefix_query_tokens = 0             # tokens of the requests that were looked up
        self.groups: List[CacheGroup] = []
        self.slot_group: Dict[int, int] = {}
        self.state_needs: Dict[int, CacheNeed] = {}
        by_key: Dict[Tuple, CacheGroup] = {}
        for slot in sorted(needs):
            need = needs[slot]
            if need.kind == "state":
                self.state_needs[slot] = need
                continue
            if need.kind != "pages":
                raise ValueError(f"cache slot {slot}: unknown cache need kind '{need.kind}'")
            if need.window is not None and need.window <= 0:
                raise ValueError(f"cache slot {slot}: window must be positive")
            k = need.group_key()
            g = by_key.get(k)
            if g is None:
                g = CacheGroup(len(self.groups), k, need.window, need.entries, [])
                n = num_pages[k] if isinstance(num_pages, dict) else num_pages
                g.pool = PagePool(n)
                by_key[k] = g
                self.groups.append(g)
            g.slots.append(slot)
            self.slot_group[slot] = g.index
        self.state_slots = StateSlots(max_requests)
        self.admit_hooks = []                    # called with the state slot of every request that is admitted
        self.requests: Dict[Hashable, RequestCache] = {}
        if prefix_caching and (len(self.groups) != 1 or self.groups[0].window is not None or self.state_needs):
            raise ValueError("prefix caching needs a model whose layers all keep all keys in pages of one kind "
                             "and no per-request state")

    # ------------------------------------------------------------------ queries

    def _first_needed_page(self, g: CacheGroup, committed: int) -> int:
        """Logical page below which no later query of the request can look."""
        if g.window is None:
            return 0
        first_pos = committed - g.window + 1   # oldest key the next query (at `committed`) sees
        return max(0, first_pos) // self.page_size

    def pages_to_extend(self, rid: Optional[Hashable], n_tokens: int) -> Dict[int, int]:
        """Pages each group must give so that positions [0, n_tokens) of the request are held."""
        rc = self.requests.get(rid) if rid is not None else None
        out = {}
        n_logical = -(-n_tokens // self.page_size)
        for g in self.groups:
            if rc is None:
                out[g.index] = n_logical - self._first_needed_page(g, 0)
            else:
                have = len(rc.tables[g.index])
                out[g.index] = max(0, n_logical - have)
        return out

    def can_extend(self, rid: Optional[Hashable], n_tokens: int) -> bool:
        if rid is None or rid not in self.requests:
            if self.state_slots.num_free == 0:
                return False
        need = self.pages_to_extend(rid, n_tokens)
        return all(self.groups[gi].pool.num_free >= n for gi, n in need.items())

    def peak_pages(self, n_tokens: int, max_portion: int) -> Dict[int, int]:
        """Most pages a request of n_tokens holds at once in each group, when no step brings
        more than max_portion of its tokens: all of them without a window, else the portion
        plus the window (and the partial pages at both ends)."""
        n_logical = -(-n_tokens // self.page_size)
        out = {}
        for g in self.groups:
            if g.window is None:
                out[g.index] = n_logical
            else:
                span = min(n_tokens, max_portion) + g.window - 1
                out[g.index] = min(n_logical, -(-span // self.page_size) + 1)
        return out

    def fits_at_all(self, n_tokens: int, max_portion: int) -> bool:
        """Whether an otherwise empty cache could hold a request of this length."""
        peak = self.peak_pages(n_tokens, max_portion)
        return all(peak[g.index] <= g.pool.num_pages for g in self.groups)

    def can_admit(self, n_tokens: int, max_portion: int) -> bool:
        """Whether a new request of this length can be taken in now: a state slot is free and
        every group has, free at this moment, the most pages the request will hold at once."""
        if self.state_slots.num_free == 0:
            return False
        peak = self.peak_pages(n_tokens, max_portion)
        return all(g.pool.num_free >= peak[g.index] for g in self.groups)

    # ------------------------------------------------------------------ life of a request

    def admit(self, rid: Hashable) -> RequestCache:
        if rid in self.requests:
            raise RuntimeError(f"request {rid!r} is already admitted")
        rc = RequestCache(state_slot=self.state_slots.allocate(rid))
        for g in self.groups:
            rc.tables[g.index] = []
        self.requests[rid] = rc
        for hook in self.admit_hooks:      # the storage clears the slot's state: a request starts from zeros
            hook(rc.state_slot)
        return rc

    def extend(self, rid: Hashable, n_tokens: int) -> None:
        """Makes room for positions [0, n_tokens).  All or nothing: raises OutOfPages and
        leaves the request as it was if any group cannot give its pages."""
        rc = self.requests[rid]
        if n_tokens < rc.committed:
            raise ValueError("a request cannot shrink")
        need = self.pages_to_extend(rid, n_tokens)
        for gi, n in need.items():
            if self.groups[gi].pool.num_free < n:
                raise OutOfPages(
                    f"request {rid!r}: group {gi} needs {n} pages, {self.groups[gi].pool.num_free} free"
                )
        for gi, n in need.items():
            if n:
                rc.tables[gi].extend(self.groups[gi].pool.allocate(n, (rid, gi)))
        rc.reserved = max(rc.reserved, n_tokens)

    def commit(self, rid: Hashable, n_tokens: int) -> None:
        """The step that brought the request to n_tokens has run."""
        rc = self.requests[rid]
        if n_tokens < rc.committed:
            raise ValueError(f"request {rid!r}: commit({n_tokens}) below what is committed")
        for g in self.groups:
            if n_tokens > len(rc.tables[g.index]) * self.page_size:
                raise ValueError(f"request {rid!r}: commit({n_tokens}) beyond what was reserved")
        rc.committed = n_tokens
        for g in self.groups:
            if g.window is None:
                continue
            table = rc.tables[g.index]
            first = min(self._first_needed_page(g, n_tokens), len(table))
            gone = [p for p in table[:first] if p != NO_PAGE]
            if gone:
                g.pool.free(gone, (rid, g.index))
                for i in range(first):
                    table[i] = NO_PAGE

    def release(self, rid: Hashable) -> None:
        rc = self.requests.pop(rid)
        for g in self.groups:
            held = [p for p in rc.tables[g.index] if p != NO_PAGE]
            # Freed in reverse so that the lowest ids are handed out first again
            # (atom/model_engine/block_manager.py:1083-1107 frees in reverse order too).
            g.pool.free(reversed(held), (rid, g.index))
        self.state_slots.free(rc.state_slot)

    # ------------------------------------------------------------------ prefix caching

    def _key(self, parent: Optional[int], tokens: Tuple[int, ...], make: bool) -> Optional[int]:
        pair = (parent, tokens)
        k = self._chains.get(pair)
        if k is None and make:
            k = self._next_key
            self._next_key += 1
            self._chains[pair] = k
            self._chain_of[k] = pair
        return k

    def claim_prefix(self, rid: Hashable, tokens) -> int:
        """For a request that has just been admitted: takes the published pages that hold the
        beginning of ``tokens`` (all but the last token at most) and returns how many tokens they
        cover; the request continues behind them."""
        if not self.prefix_caching:
            return 0
        rc = self.requests[rid]
        if rc.committed or rc.tables[0]:
            raise RuntimeError(f"request {rid!r} already holds pages")
        pool, ps = self.groups[0].pool, self.page_size
        self.prefix_query_tokens += len(tokens)
        parent, n = None, 0
        while (n + 1) * ps <= len(tokens) - 1:
            key = self._key(parent, tuple(tokens[n * ps:(n + 1) * ps]), make=False)
            page = pool.lookup(key) if key is not None else None
            if page is None:
                break
            pool.share(page, (rid, 0))
            rc.tables[0].append(page)
            parent = key
            n += 1
        rc.published, rc.chain = n, parent
        rc.committed = rc.reserved = n * ps
        self.prefix_hit_tokens += n * ps
        return n * ps

    def publish(self, rid: Hashable, tokens) -> None:
        """After a step: the request's pages that are full of committed tokens become findable.
        ``tokens``: the request's tokens from its first one (at least the committed ones)."""
        if not self.prefix_caching or rid not in self.requests:
            return
        rc = self.requests[rid]
        pool, ps = self.groups[0].pool, self.page_size
        while (rc.published + 1) * ps <= rc.committed:
            i = rc.published
            key = self._key(rc.chain, tuple(tokens[i * ps:(i + 1) * ps]), make=True)
            pool.publish(rc.tables[0][i], key)     # (no effect if another page already answers to the key)
            rc.chain = key
            rc.published += 1
        self._forget_dead_keys()

    def _forget_dead_keys(self) -> None:
        """Keys whose page was given up are of no use; dropped in bulk now and then."""
        pool = self.groups[0].pool
        if len(self._chain_of) <= 2 * pool.num_pages + 1024:
            return
        for k in [k for k in self._chain_of if pool.lookup(k) is None]:
            del self._chains[self._chain_of.pop(k)]

    # ------------------------------------------------------------------ views

    def table(self, rid: Hashable, group: int) -> List[int]:
        return self.requests[rid].tables[group]

    def committed(self, rid: Hashable) -> int:
        return self.requests[rid].committed

    def num_free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free

    def check(self) -> None:
        """Accounting invariants: no page lost, held twice or by a request that is gone."""
        self.state_slots.check()
        for g in self.groups:
            g.pool.check()
            seen = set()
            for rid, rc in self.requests.items():
                for p in rc.tables[g.index]:
                    if p == NO_PAGE:
                        continue
                    if p in seen and not self.prefix_caching:
                        raise AssertionError(f"page {p} of group {g.index} is in two tables")
                    seen.add(p)
                    if (rid, g.index) not in g.pool.holders_of(p):
                        raise AssertionError(f"page {p} of group {g.index}: owner mismatch")
                if len(set(q for q in rc.tables[g.index] if q != NO_PAGE)) != sum(q != NO_PAGE for q in rc.tables[g.index]):
                    raise AssertionError(f"request {rid!r} holds a page of group {g.index} twice")
            if self.prefix_caching:
                held = sum(len(g.pool.holders_of(p)) for p in seen)
                in_tables = sum(sum(q != NO_PAGE for q in rc.tables[g.index]) for rc in self.requests.values())
                if held != in_tables:
                    raise AssertionError(f"group {g.index}: {held} holdings, {in_tables} table entries")
            if len(seen) != g.pool.num_used:
                raise AssertionError(f"group {g.index}: {g.pool.num_used} pages held, {len(seen)} in tables")
