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
