"""The cache manager: pages, block tables, groups with and without a window, state slots."""

from __future__ import annotations

import random

import pytest

from inference_engine_b200.cache import (
    CacheManager, OutOfPages, PagedGroupSpec, PagePool, SlotPool, StateGroupSpec,
)


def _manager(num_pages=8, page_size=4, window=None, max_requests=4, state=False):
    groups = [PagedGroupSpec(2, 2, 16, None)]
    if window:
        groups.append(PagedGroupSpec(1, 1, 32, window))
    return CacheManager(groups, [StateGroupSpec(1, (8,))] if state else [], num_pages, page_size, max_requests)


def test_page_pool_is_first_in_first_out_and_strict():
    pool = PagePool(3)
    assert [pool.allocate() for _ in range(3)] == [0, 1, 2]
    with pytest.raises(OutOfPages):
        pool.allocate()
    pool.free(1)
    pool.free(0)
    assert pool.num_free == 2
    with pytest.raises(ValueError, match="double free"):
        pool.free(0)
    with pytest.raises(ValueError, match="does not exist"):
        pool.free(7)
    with pytest.raises(ValueError, match="cannot be shared"):
        pool.incref(1)
    assert [pool.allocate(), pool.allocate()] == [1, 0]  # given back first, handed out first
    pool.incref(2)
    pool.free(2)
    assert pool.refcount(2) == 1 and pool.num_free == 0


def test_slot_pool():
    slots = SlotPool(2)
    a, b = slots.allocate(), slots.allocate()
    with pytest.raises(OutOfPages):
        slots.allocate()
    slots.free(a)
    with pytest.raises(ValueError, match="double free"):
        slots.free(a)
    assert slots.allocate() == a and slots.used_slots() == {a, b}


def test_grow_slot_math_and_free():
    m = _manager()
    m.add_request("a")
    assert m.pages_needed("a", 0, 9) == [3]
    m.grow("a", 0, 9)
    assert m.table(0, "a") == [0, 1, 2] and m.num_free_pages == [5]
    assert m.slot(0, "a", 0) == 0 and m.slot(0, "a", 5) == 1 * 4 + 1 and m.slot(0, "a", 8) == 2 * 4
    m.grow("a", 9, 12)  # still inside the third page
    assert m.table(0, "a") == [0, 1, 2]
    m.grow("a", 12, 13)
    assert m.table(0, "a") == [0, 1, 2, 3]
    assert not m.can_grow("a", 13, 13 + 4 * 5)
    with pytest.raises(OutOfPages):
        m.grow("a", 13, 13 + 4 * 5)
    assert m.table(0, "a") == [0, 1, 2, 3]  # a failed grow changes nothing
    m.check_invariants()
    m.free("a")
    assert m.num_free_pages == [8] and not m.has_request("a")
    m.free("a")  # freeing twice is harmless at this level: the request is gone
    m.add_request("b")
    with pytest.raises(ValueError, match="already"):
        m.add_request("b")


def test_pages_are_used_again_by_later_requests():
    m = _manager(num_pages=4)
    m.add_request("a")
    m.grow("a", 0, 16)
    m.add_request("b")
    assert not m.can_grow("b", 0, 1)
    m.free("a")
    m.grow("b", 0, 7)
    assert m.table(0, "b") == [0, 1]
    m.check_invariants()


def test_window_group_takes_and_gives_back_pages():
    m = _manager(num_pages=6, page_size=4, window=6)
    m.add_request("a")
    m.grow("a", 0, 14)  # a 14-token portion: every page of it is needed during the step
    assert [len(m.table(g, "a")) for g in (0, 1)] == [4, 4]
    assert m.release_behind_window("a", 14) == 2  # next query at 14 sees 9..14: pages 0, 1 go
    assert m.table(1, "a") == [-1, -1, 2, 3] and m.table(0, "a") == [0, 1, 2, 3]
    assert m.num_free_pages == [2, 4]
    with pytest.raises(ValueError, match="no longer cached"):
        m.slot(1, "a", 3)
    for pos in range(14, 24):  # decode: the windowed group never holds more than 3 pages
        m.grow("a", pos, pos + 1)
        m.release_behind_window("a", pos + 1)
        assert len([p for p in m.table(1, "a") if p >= 0]) <= 3
        m.check_invariants()
    assert m.table(0, "a") == [0, 1, 2, 3, 4, 5]
    assert not m.can_grow("a", 24, 25)  # the group that keeps everything is full
    m.free("a")
    assert m.num_free_pages == [6, 6]


def test_window_group_only_needs_pages_the_next_queries_see():
    m = _manager(num_pages=3, page_size=4, window=4)
    m.add_request("a")
    with pytest.raises(OutOfPages):  # the full group needs 5 pages
        m.grow("a", 0, 20)
    m2 = CacheManager([PagedGroupSpec(1, 1, 16, 4)], [], 3, 4, 2)
    m2.add_request("a")
    pos = 0
    for n in (8, 8, 8, 8):  # portions of 8 with a window of 4: at most 3 pages at a time
        m2.grow("a", pos, pos + n)
        pos += n
        m2.release_behind_window("a", pos)
        m2.check_invariants()
    assert m2.table(0, "a")[:7] == [-1] * 7


def test_state_slots_follow_the_requests():
    m = _manager(max_requests=2, state=True)
    a, b = m.add_request("a"), m.add_request("b")
    assert {a, b} == {0, 1} and not m.can_admit()
    with pytest.raises(OutOfPages):
        m.add_request("c")
    m.free("a")
    assert m.can_admit() and m.add_request("c") == a
    m.check_invariants()


def test_recompute_preemption_gives_back_pages_but_keeps_the_request():
    m = _manager()
    m.add_request("a")
    m.grow("a", 0, 10)
    m.release_pages("a")
    assert m.num_free_pages == [8] and m.has_request("a") and m.table(0, "a") == []
    m.grow("a", 0, 3)
    m.check_invariants()


@pytest.mark.parametrize("seed", range(8))
def test_no_page_lost_held_twice_or_freed_twice_under_random_orders(seed):
    rng = random.Random(seed)
    window = rng.choice([None, 5, 9])
    m = _manager(num_pages=rng.randint(6, 20), page_size=rng.choice([1, 2, 4, 8]), window=window,
                 max_requests=5, state=True)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.can_admit():
            m.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.75 and live:
            rid = rng.choice(list(live))
            n = rng.randint(1, 12)
            if m.can_grow(rid, live[rid], live[rid] + n):
                m.grow(rid, live[rid], live[rid] + n)
                live[rid] += n
                m.release_behind_window(rid, live[rid])
            else:
                with pytest.raises(OutOfPages):
                    m.grow(rid, live[rid], live[rid] + n)
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            m.release_pages(rid)
            live[rid] = 0
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check_invariants()
        # every position a later query can see maps to a page, and no two live positions share a slot
        seen = [set() for _ in m.pools]
        for rid, n in live.items():
            for g, spec in enumerate(m.paged_groups):
                first = 0 if spec.window is None else max(n - spec.window + 1, 0)
                for pos in range(first, n):
                    slot = m.slot(g, rid, pos)
                    assert slot not in seen[g]
                    seen[g].add(slot)
    for rid in list(live):
        m.free(rid)
    assert m.num_free_pages == [p.num_pages for p in m.pools] and m.slots.num_free == 5
