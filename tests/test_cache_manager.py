"""The cache manager on the CPU: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; slots come and go with pages."""

import random

import pytest

from servelab_b200.cache import CacheError, CacheManager, PagePool, StateSlotPool


def test_grow_release_fifo_and_slot_formula():
    m = CacheManager([None], 8, 4, num_state_slots=2)
    assert m.open("a") and m.ensure("a", 6)
    assert m.block_table("a", 0) == [0, 1]
    assert m.ensure("a", 8) and m.block_table("a", 0) == [0, 1]      # still fits
    assert m.ensure("a", 9) and m.block_table("a", 0) == [0, 1, 2]
    p, bs = 6, 4
    assert m.block_table("a", 0)[p // bs] * bs + p % bs == 6
    assert m.open("b") and m.ensure("b", 4) and m.block_table("b", 0) == [3]
    m.release("a")
    assert list(m.pools[0].free) == [4, 5, 6, 7, 0, 1, 2]            # FIFO reuse
    m.release("a")                                                     # twice: harmless
    m.check_invariants()
    with pytest.raises(CacheError):
        m.open("b")                                                    # already open


def test_all_groups_or_nothing():
    m = CacheManager([None, None], [4, 2], 4, num_state_slots=4)
    assert m.open("a")
    assert not m.ensure("a", 12)            # group 1 has only 2 pages
    assert m.block_table("a", 0) == [] and m.block_table("a", 1) == []
    assert m.alloc_fails == 1
    assert m.ensure("a", 8)
    assert not m.can_ever_hold(12, 4) and m.can_ever_hold(8, 4)
    m.check_invariants()


def test_window_pages_are_given_back_and_reused():
    m = CacheManager([None, 6], 16, 4, num_state_slots=2)
    assert m.open("a")
    for n in range(1, 41):
        assert m.ensure("a", n)
        m.trim("a", n)                      # next query sits at position n
        full, win = m.block_table("a", 0), m.block_table("a", 1)
        assert all(p >= 0 for p in full) and len(full) == -(-n // 4)
        # keys the next query needs: n - 6 + 1 .. n ; their pages must be live
        for r in range(max(0, n - 5), n):
            assert win[r // 4] >= 0, (n, r)
        # pages wholly behind the window are gone
        for lp in range(len(win)):
            if (lp + 1) * 4 <= n - 5:
                assert win[lp] == -1, (n, lp)
    assert sum(1 for p in m.block_table("a", 1) if p >= 0) <= 3
    m.check_invariants()
    m.release("a")
    m.check_invariants()
    assert m.pools[1].num_free() == 16
    assert m.pools[1].peak_pages(1000, 8) == 5


def test_state_slots():
    s = StateSlotPool(2)
    assert s.take("a") == 0 and s.take("b") == 1 and s.take("c") is None
    assert s.drain_to_clear() == [0, 1] and s.drain_to_clear() == []
    assert s.give("a") == 0 and s.give("a") is None
    assert s.take("c") == 0 and s.drain_to_clear() == [0]
    m = CacheManager([None], 4, 4, num_state_slots=1)
    assert m.open("a") and not m.open("b")
    m.release("a")
    assert m.open("b") and m.state_slot("b") == 0


def test_reserve_only_limits_admission():
    m = CacheManager([None], 4, 4, num_state_slots=4, reserve_pages=1)
    assert m.open("a")
    assert not m.ensure("a", 16, for_admission=True)
    assert m.ensure("a", 12, for_admission=True)
    assert m.ensure("a", 16)                 # a running request may use the reserve
    assert not m.can_ever_hold(16, 16) and m.can_ever_hold(12, 16)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_never_lose_or_duplicate_pages(seed):
    rng = random.Random(seed)
    windows = [None, rng.choice([5, 9, 16])]
    m = CacheManager(windows, [rng.randint(6, 20), rng.randint(6, 20)], rng.choice([2, 4, 8]),
                     num_state_slots=3)
    live = {}
    for step in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{step}"
            if m.open(rid):
                live[rid] = 0
            else:
                assert m.slots.num_free() == 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = live[rid] + rng.randint(1, 9)
            free_before = [p.num_free() for p in m.pools]
            if m.ensure(rid, n):
                live[rid] = n
                m.trim(rid, n)
            else:
                assert [p.num_free() for p in m.pools] == free_before     # nothing changed
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
            if rng.random() < 0.3:
                m.release(rid)
        m.check_invariants()
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert all(p.num_free() == p.num_pages for p in m.pools) and m.slots.num_free() == 3


def test_invariant_check_catches_a_double_free():
    p = PagePool(4, 4)
    p.open("a")
    p.grow("a", 8)
    table = list(p.tables["a"])
    p.close("a")
    p.free.extend(table)                     # simulate a page freed twice
    m = CacheManager([None], 4, 4, 1)
    m.pools[0] = p
    with pytest.raises(CacheError):
        m.check_invariants()
