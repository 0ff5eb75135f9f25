"""The cache manager on the CPU: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots are accounted the same way."""
import random

import pytest

from atom_b200.cache import NO_PAGE, CacheManager, OutOfPages, OutOfSlots, PagePool, StateSlots
from atom_b200.parts.spec import CacheNeed

FULL = CacheNeed("pages", num_kv_heads=2, head_dim=16)
WIN = CacheNeed("pages", num_kv_heads=2, head_dim=16, window=20)
OTHER = CacheNeed("pages", num_kv_heads=1, head_dim=32)
STATE = CacheNeed("state", state_shape=(4, 3))


def test_pool_lowest_first_and_reuse():
    p = PagePool(5)
    a = p.allocate(3, "a")
    assert a == [0, 1, 2]
    p.free([1], "a")
    assert p.allocate(2, "b") == [1, 3]
    p.check()
    with pytest.raises(OutOfPages):
        p.allocate(2, "c")
    assert p.num_free == 1          # nothing was taken by the failed call
    with pytest.raises(RuntimeError):
        p.free([1], "a")            # held by b
    p.free([1, 3], "b")
    with pytest.raises(RuntimeError):
        p.free([3])                 # freed twice
    with pytest.raises(RuntimeError):
        p.free([0, 0])
    p.check()


def test_state_slots():
    s = StateSlots(2)
    a, b = s.allocate("x"), s.allocate("y")
    assert (a, b) == (0, 1)
    with pytest.raises(OutOfSlots):
        s.allocate("z")
    s.free(a)
    with pytest.raises(RuntimeError):
        s.free(a)
    assert s.allocate("z") == 0
    s.check()


def test_groups_by_need():
    m = CacheManager({0: FULL, 1: WIN, 2: FULL, 3: OTHER, 4: STATE, 5: WIN}, 8, 10, 4)
    assert [g.slots for g in m.groups] == [[0, 2], [1, 5], [3]]
    assert m.slot_group == {0: 0, 2: 0, 1: 1, 5: 1, 3: 2}
    assert list(m.state_needs) == [4]


def test_extend_commit_release_and_block_table():
    m = CacheManager({0: FULL}, 8, 6, 2)
    m.admit("a")
    m.extend("a", 17)
    assert m.table("a", 0) == [0, 1, 2]
    m.commit("a", 17)
    m.extend("a", 24)               # still inside the third page
    assert m.table("a", 0) == [0, 1, 2]
    m.extend("a", 25)
    assert m.table("a", 0) == [0, 1, 2, 3]
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.extend("b", 17)           # needs 3, 2 free
    assert m.table("b", 0) == [] and m.num_free_pages(0) == 2   # all or nothing
    m.check()
    m.release("a")
    m.extend("b", 17)
    assert m.table("b", 0) == [0, 1, 2]                         # freed pages are used again
    with pytest.raises(ValueError):
        m.commit("b", 30)           # beyond what was reserved
    m.release("b")
    m.check()
    assert m.num_free_pages(0) == 6 and m.state_slots.num_free == 2


def test_window_gives_pages_back():
    m = CacheManager({0: FULL, 1: WIN}, 8, 12, 2)
    m.admit("a")
    m.extend("a", 30)
    m.commit("a", 30)               # next query at 30 sees keys >= 11: page 0 (0..7) has passed
    assert m.table("a", 1) == [NO_PAGE, 1, 2, 3] and m.table("a", 0) == [0, 1, 2, 3]
    for n in range(31, 80):
        m.extend("a", n)
        m.commit("a", n)
        live = [p for p in m.table("a", 1) if p != NO_PAGE]
        first_needed = max(0, n - 20 + 1) // 8
        assert m.table("a", 1)[:first_needed] == [NO_PAGE] * first_needed
        assert len(live) <= 4       # window 20 over pages of 8: at most 4 pages
        m.check()
    assert len(m.table("a", 0)) == 10
    m.release("a")
    assert m.num_free_pages(0) == 12 and m.num_free_pages(1) == 12


def test_admission_helpers():
    m = CacheManager({0: FULL, 1: WIN}, 8, 6, 1)
    assert m.peak_pages(100, 16) == {0: 13, 1: 6}
    assert not m.fits_at_all(100, 16) and m.fits_at_all(48, 16)
    assert m.can_admit(48, 16)
    m.admit("a")
    assert not m.can_admit(8, 8)    # no state slot left
    with pytest.raises(RuntimeError):
        m.admit("a")


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = CacheManager({0: FULL, 1: WIN, 2: FULL}, page_size=rng.choice([4, 8, 16]), num_pages=40, max_requests=6)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.state_slots.num_free:
            rid = f"r{next_id}"
            next_id += 1
            m.admit(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            target = live[rid] + rng.choice([1, 1, 1, 2, 5, 13, 40])
            try:
                m.extend(rid, target)
            except OutOfPages:
                before = {g.index: g.pool.num_free for g in m.groups}
                m.check()
                assert before == {g.index: g.pool.num_free for g in m.groups}
                victim = rng.choice(list(live))
                m.release(victim)
                del live[victim]
                continue
            if rng.random() < 0.9:      # a step may also be reserved and never run
                m.commit(rid, target)
                live[rid] = target
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        held = [p for rc in m.requests.values() for p in rc.tables[0] if p != NO_PAGE]
        assert len(held) == len(set(held))
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.groups)
    assert m.state_slots.num_free == 6


# ----------------------------------------------------------------------------- prefix caching


def _run(c, rid, tokens, upto):
    """Stands in for steps that compute the request's tokens up to ``upto``."""
    c.extend(rid, upto)
    c.commit(rid, upto)
    c.publish(rid, tokens)


def test_prefix_pages_are_published_claimed_shared_and_evicted_last_released_last():
    c = CacheManager({0: FULL}, page_size=4, num_pages=6, max_requests=4, prefix_caching=True)
    pool = c.groups[0].pool
    a = list(range(100, 110))                       # 10 tokens: two full pages and a half
    c.admit("a")
    assert c.claim_prefix("a", a) == 0
    _run(c, "a", a, 10)
    pa = c.table("a", 0)
    assert [pool.key_of(p) is not None for p in pa] == [True, True, False]
    c.release("a")
    assert pool.num_free == 6 and pool.num_cached == 2 and pool.num_used == 0
    c.check()
    # b begins like a (9 tokens), c like both; a request of exactly 8 tokens may take one page only
    b = a[:9] + [7, 8, 9]
    c.admit("b")
    assert c.claim_prefix("b", b) == 8 and c.table("b", 0) == pa[:2] and c.committed("b") == 8
    c.admit("c")
    assert c.claim_prefix("c", a[:8]) == 4 and c.table("c", 0) == pa[:1]
    assert sorted(pool.holders_of(pa[0])) == [("b", 0), ("c", 0)]
    c.check()
    _run(c, "b", b, 12)                             # its third page is published under another key than a's would be
    _run(c, "c", a[:8], 8)                          # c computes the page b already holds: not published twice
    assert pool.key_of(c.table("c", 0)[1]) is None
    c.release("c")
    c.release("b")
    c.check()
    assert pool.num_cached == 3 and pool.num_free == 6
    # the pool gives vacant pages first, then the cached ones, least recently released first
    c.admit("d")
    c.extend("d", 12)                               # 3 vacant pages
    assert pool.num_cached == 3 and pool.num_evictions == 0
    c.extend("d", 16)                               # the 4th evicts b's last page (released first, in reverse order)
    assert pool.num_evictions == 1 and pool.num_cached == 2
    c.admit("e")
    assert c.claim_prefix("e", b) == 8              # the first two pages are still there, the third is gone
    c.check()
    c.release("d")
    c.release("e")
    c.check()
    assert c.prefix_hit_tokens == 8 + 4 + 8


def test_prefix_caching_is_refused_where_it_cannot_hold():
    with pytest.raises(ValueError):
        CacheManager({0: FULL, 1: WIN}, 4, 8, 2, prefix_caching=True)
    with pytest.raises(ValueError):
        CacheManager({0: FULL, 1: STATE}, 4, 8, 2, prefix_caching=True)
    c = CacheManager({0: FULL}, 4, 8, 2)            # off: nothing is ever claimed or published
    c.admit("a")
    assert c.claim_prefix("a", list(range(20))) == 0
    _run(c, "a", list(range(20)), 20)
    assert c.groups[0].pool.key_of(c.table("a", 0)[0]) is None


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_with_shared_prefixes_keep_the_books(seed):
    rng = random.Random(seed)
    c = CacheManager({0: FULL}, page_size=4, num_pages=24, max_requests=5, prefix_caching=True)
    stems = [[rng.randrange(50) for _ in range(rng.randrange(4, 30))] for _ in range(3)]
    live, next_id = {}, 0
    for _ in range(400):
        op = rng.random()
        if op < 0.35 and len(live) < 5:
            toks = list(rng.choice(stems))[: rng.randrange(2, 30)] + [rng.randrange(50) for _ in range(rng.randrange(0, 6))]
            if c.can_admit(len(toks) + 1, 64):
                rid = next_id
                next_id += 1
                c.admit(rid)
                hit = c.claim_prefix(rid, toks)
                assert hit % 4 == 0 and hit <= len(toks) - 1
                # what was claimed holds the same tokens under the same keys
                live[rid] = [toks, hit]
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            toks, done = live[rid]
            if done < len(toks):
                upto = min(len(toks), done + rng.randrange(1, 9))
                try:
                    c.extend(rid, upto)
                except OutOfPages:
                    continue
                c.commit(rid, upto)
                c.publish(rid, toks)
                live[rid][1] = upto
            else:
                toks.append(rng.randrange(50))       # a decoded token
        elif live:
            rid = rng.choice(list(live))
            c.release(rid)
            del live[rid]
        c.check()
    for rid in list(live):
        c.release(rid)
    c.check()
    pool = c.groups[0].pool
    assert pool.num_used == 0 and pool.num_free == 24


def test_groups_follow_the_declared_entries_and_storage_allocates_them():
    """A mixer names what it keeps per token; slots that keep the same arrays share a group and a block
    table, others get a pool of their own, and the storage allocates exactly the declared arrays with the
    page's tokens before the last axis."""
    import torch

    from atom_b200.cache.storage import CacheStorage
    from atom_b200.parts.spec import CacheEntry

    latent = CacheNeed("pages", entries=(CacheEntry("latent", (12,), "float32"),))
    kv_unequal = CacheNeed("pages", entries=(CacheEntry("k", (2, 24)), CacheEntry("v", (2, 16))))
    assert FULL.entries == (CacheEntry("k", (2, 16)), CacheEntry("v", (2, 16)))
    m = CacheManager({0: FULL, 1: latent, 2: FULL, 3: kv_unequal, 4: latent}, page_size=8, num_pages=5, max_requests=2)
    assert [g.slots for g in m.groups] == [[0, 2], [1, 4], [3]]
    st = CacheStorage(m, torch.bfloat16, "cpu")
    v0, v1, v3 = st.view(0), st.view(1), st.view(3)
    assert v0.k_pages.shape == (5, 2, 8, 16) and v0.v_pages.dtype == torch.bfloat16 and v0.group == 0
    assert set(v1.pages) == {"latent"} and v1.pages["latent"].shape == (5, 8, 12) and v1.k_pages is None
    assert v1.pages["latent"].dtype == torch.float32 and v1.group == 1
    assert v3.pages["k"].shape == (5, 2, 8, 24) and v3.pages["v"].shape == (5, 2, 8, 16)
    assert st.view(2).k_pages.data_ptr() != v0.k_pages.data_ptr()
    per_page = 2 * (2 * 2 * 16 * 8 * 2) + 2 * (12 * 8 * 4) + (2 * 24 + 2 * 16) * 8 * 2
    assert CacheStorage.bytes_per_page(m, torch.bfloat16) == per_page
    assert st.bytes() == 5 * per_page
    with pytest.raises(ValueError):
        CacheNeed("pages")
    with pytest.raises(ValueError):
        CacheNeed("pages", entries=(CacheEntry("a", (4,)), CacheEntry("a", (4,))))
