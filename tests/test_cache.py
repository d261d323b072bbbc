"""The cache manager's bookkeeping (CPU): no page lost, held twice or freed twice."""
import random

import pytest

from infinicore_infer_b200.cache import (NO_PAGE, CacheGroup, CacheManager, OutOfPages, OutOfSlots,
                                          PagedKV, PagePool, SlotAllocator, StateSlot)


def test_pool_hands_out_each_page_once_and_reuses_the_last_freed():
    pool = PagePool(9, reserved=1)
    assert pool.capacity == 8 and pool.available == 8
    a = pool.alloc(3)
    assert a == [1, 2, 3] and 0 not in a
    b = pool.alloc(5)
    assert sorted(a + b) == list(range(1, 9))
    with pytest.raises(OutOfPages):
        pool.alloc(1)
    pool.free([2])
    pool.free([7, 5])
    assert pool.alloc(1) == [5]            # last freed, first used again
    assert pool.alloc(2) == [7, 2]
    assert pool.high_water == 8


def test_pool_refuses_double_free_foreign_and_null_pages():
    pool = PagePool(5, reserved=1)
    p = pool.alloc(2)
    pool.free([p[0]])
    with pytest.raises(ValueError, match="freed twice"):
        pool.free([p[0]])
    with pytest.raises(ValueError, match="not one of"):
        pool.free([0])
    with pytest.raises(ValueError, match="not one of"):
        pool.free([99])
    with pytest.raises(ValueError, match="twice in one free"):
        pool.free([p[1], p[1]])
    with pytest.raises(ValueError):
        pool.free([3])                      # never handed out
    assert pool.in_use == 1


def test_out_of_pages_takes_nothing():
    pool = PagePool(4, reserved=1)
    pool.alloc(2)
    with pytest.raises(OutOfPages) as e:
        pool.alloc(2)
    assert e.value.wanted == 2 and e.value.available == 1
    assert pool.available == 1


def _manager(num_pages=8, page=4, window=None, max_requests=4, max_positions=64, state=False):
    needs = [PagedKV(2, 16, None), PagedKV(2, 16, window), PagedKV(2, 16, None)]
    if state:
        needs.append(StateSlot((4,)))
    return CacheManager(needs, num_pages, page, max_requests, max_positions, device=None)


def test_layers_with_equal_needs_share_a_group_and_windows_get_their_own():
    m = _manager(window=6)
    assert len(m.groups) == 2
    assert m.groups[0].cache_ids == [0, 2] and m.groups[1].cache_ids == [1]
    assert m.views[0].group_index == m.views[2].group_index == 0 and m.views[1].group_index == 1
    assert len(_manager(window=None).groups) == 1


def test_reserve_commit_release_cycle():
    m = _manager(num_pages=6, page=4)
    m.admit("a")
    assert m.pages_needed("a", 5) == [2]
    m.reserve("a", 5)
    m.commit("a", 5)
    assert m.length("a") == 5 and m.groups[0].pool.in_use == 2
    assert m.pages_needed("a", 8) == [0]        # the second page has room for positions 5..7
    m.reserve("a", 9)
    m.commit("a", 9)
    assert m.groups[0].pool.in_use == 3
    table = list(m.groups[0].table("a"))
    assert len(table) == 3 and NO_PAGE not in table and len(set(table)) == 3
    m.check_invariants()
    m.release("a")
    assert m.groups[0].pool.in_use == 0 and not m.is_live("a")
    with pytest.raises(KeyError):
        m.release("a")
    m.check_invariants()


def test_reserve_is_all_or_nothing_across_groups():
    m = CacheManager([PagedKV(1, 16), PagedKV(1, 32)], 4, 4, 4, 64, device=None, pages_per_group={1: 2})
    m.admit("a")
    assert not m.can_reserve({"a": 12})
    with pytest.raises(OutOfPages):
        m.reserve("a", 12)                  # group 0 has the 3 pages, group 1 only 2
    assert all(g.pool.in_use == 0 for g in m.groups)
    m.check_invariants()
    assert m.can_reserve({"a": 8})
    m.reserve("a", 8)
    m.check_invariants()


def test_can_reserve_counts_all_requests_of_a_step_together():
    m = _manager(num_pages=4, page=4)
    m.admit("a"); m.admit("b")
    assert m.can_reserve({"a": 8}) and m.can_reserve({"b": 8})
    assert m.can_reserve({"a": 8, "b": 8})
    assert not m.can_reserve({"a": 8, "b": 9})


def test_context_overflow_is_refused():
    m = _manager(max_positions=16)
    m.admit("a")
    with pytest.raises(ValueError, match="exceed"):
        m.reserve("a", 17)


def test_window_group_gives_passed_pages_back():
    page, window = 4, 6
    m = CacheManager([PagedKV(1, 16, window)], 5, page, 2, 256, device=None)
    g = m.groups[0]
    m.admit("a")
    pos = 0
    peak = 0
    for step_len in [3, 2, 7, 1, 1, 1, 9, 2] + [1] * 40:
        m.reserve("a", pos + step_len)
        peak = max(peak, g.pool.in_use)
        # every block a query of this step can see is present
        lo = max(0, pos - window + 1)
        table = g.table("a")
        for b in range(lo // page, (pos + step_len - 1) // page + 1):
            assert table[b] != NO_PAGE
        pos += step_len
        m.commit("a", pos)
        m.check_invariants()
        # nothing below the next query's window is still held
        first_visible = max(0, pos - window + 1) // page
        assert all(p == NO_PAGE for p in g.table("a")[:first_visible])
    assert g.pool.in_use <= (window + page - 1) // page + 1
    assert peak <= 5 and pos > 60          # far more positions than the pool has pages for
    m.release("a")
    assert g.pool.in_use == 0


def test_slots():
    s = SlotAllocator(2)
    assert s.num_slots == 3
    a, b = s.acquire("a"), s.acquire("b")
    assert {a, b} == {1, 2}
    with pytest.raises(OutOfSlots):
        s.acquire("c")
    with pytest.raises(ValueError):
        s.acquire("a")
    s.release("a")
    assert s.acquire("c") == a
    with pytest.raises(ValueError):
        s.release("a")


def test_state_slot_is_part_of_a_request_even_with_no_state():
    m = _manager()
    slot = m.admit("a")
    assert slot >= 1 and m.slot_ids(["a"]) == [slot]
    m.release("a")
    assert m.slots.available == 4


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    window = rng.choice([None, 5, 11])
    page = rng.choice([2, 4, 8])
    m = CacheManager([PagedKV(2, 16, None), PagedKV(2, 16, window), PagedKV(1, 32, None)],
                     rng.randint(6, 14), page, 4, 96, device=None)
    live, next_id, refused = {}, 0, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            m.admit(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 12])
            new_len = min(96, live[r] + n)
            if new_len == live[r]:
                continue
            for g in m.groups:
                # the count without a scan equals the count by looking at every block
                t = g.table(r)
                first = max(g._first_needed_block(live[r]), g.first_block.get(r, 0))
                by_scan = sum(1 for b in range(first, (new_len + page - 1) // page) if b >= len(t) or t[b] == NO_PAGE)
                assert g.pages_needed(r, live[r], new_len) == by_scan
            ok = m.can_reserve({r: new_len})
            try:
                m.reserve(r, new_len)
                assert ok
                m.commit(r, new_len); live[r] = new_len
            except OutOfPages:
                assert not ok
                refused += 1
        elif live:
            r = rng.choice(list(live))
            m.release(r); del live[r]
        m.check_invariants()
        for g in m.groups:
            assert g.pool.in_use + g.pool.available == g.pool.capacity
            for r, n in live.items():
                t = g.table(r)
                first = 0 if g.need.window is None else max(0, n - g.need.window + 1) // page
                for b in range(first, (n + page - 1) // page):
                    assert t[b] != NO_PAGE
    for r in list(live):
        m.release(r)
    assert all(g.pool.in_use == 0 for g in m.groups)
    assert refused > 0                      # the pools were small enough to run out
