"""The cache manager's bookkeeping on the CPU: no page lost, held twice or freed twice, under
random orders of requests; all-or-nothing growth; windows give pages back; slots recycle."""
import random

import numpy as np
import pytest

from litellmengine_b200.cache import (CacheError, CacheManager, OutOfPages, PagedNeed, PagePool, StateNeed)

FULL = PagedNeed(2, 16, None)
WIN = PagedNeed(2, 16, 10)


def test_pool_order_exhaustion_and_double_free():
    p = PagePool(4)
    assert p.take(2) == [0, 1]                 # a fresh pool hands out 0, 1, 2, ...
    with pytest.raises(OutOfPages):
        p.take(3)
    assert p.free_count == 2                   # a refused request takes nothing
    p.give([1])
    assert p.take(1) == [1]                    # last in, first out
    with pytest.raises(CacheError, match="twice"):
        p.give([0, 0])
    p.give([0])
    with pytest.raises(CacheError, match="freed twice"):
        p.give([0])
    with pytest.raises(CacheError, match="outside"):
        p.give([9])


def test_address_rule_and_table_updates():
    m = CacheManager([FULL, FULL], page_size=4, max_total_tokens=32, max_slots=2)
    assert len(m.groups) == 1 and m.groups[0].stages == [0, 1]
    s = m.admit()
    m.ensure(s, 9)                             # 3 pages
    g = m.groups[0]
    assert g.held_pages(s) == [0, 1, 2] and list(g.table[s, :3]) == [0, 1, 2]
    (idx, val), = m.drain_updates()
    assert list(idx) == [s * g.max_pages_per_request + i for i in range(3)] and list(val) == [0, 1, 2]
    assert all(len(i) == 0 for i, _ in m.drain_updates())
    m.commit(s, 9)
    m.ensure(s, 12)                            # still 3 pages: nothing new
    assert all(len(i) == 0 for i, _ in m.drain_updates())
    m.ensure(s, 13)
    assert g.held_pages(s) == [0, 1, 2, 3]
    m.check_invariants()


def test_ensure_is_all_or_nothing_across_groups():
    m = CacheManager([FULL, WIN], page_size=4, max_total_tokens=16, max_slots=3)
    assert len(m.groups) == 2                  # different needs, pages of their own
    a, b = m.admit(), m.admit()
    m.ensure(a, 12)
    m.commit(a, 12)                            # window 10: positions < 3 not needed -> no whole page yet
    free_before = [g.pool.free_count for g in m.groups]
    with pytest.raises(OutOfPages):
        m.ensure(b, 8)                         # needs 2 pages, each group has 1
    assert [g.pool.free_count for g in m.groups] == free_before
    assert not m.can_hold([(b, 8)]) and m.can_hold([(b, 4)])
    assert not m.can_hold([(b, 4), (None, 1)])
    m.check_invariants()


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([WIN], page_size=4, max_total_tokens=24, max_slots=1)
    s = m.admit()
    g = m.groups[0]
    freed = 0
    for n in range(1, 25):
        m.ensure(s, n)
        freed += m.commit(s, n)
        # the next query sits at position n and sees keys n-9 .. n
        first_needed = max(0, n - 10 + 1)
        assert g.first_held[s] == first_needed // 4
        m.check_invariants()
    assert freed == g.first_held[s] == 3 and len(g.held_pages(s)) == 3
    m.release(s)
    assert g.pool.free_count == g.pool.num_pages
    m.check_invariants()


def test_limits_and_misuse():
    m = CacheManager([FULL], page_size=4, max_total_tokens=16, max_slots=1, max_request_tokens=10)
    s = m.admit()
    with pytest.raises(OutOfPages, match="no free request slot"):
        m.admit()
    with pytest.raises(OutOfPages, match="exceeds the limit"):
        m.ensure(s, 11)
    m.ensure(s, 6)
    m.commit(s, 6)
    with pytest.raises(CacheError, match="never shrinks"):
        m.commit(s, 5)
    m.release(s)
    with pytest.raises(CacheError, match="not held"):
        m.release(s)
    with pytest.raises(CacheError, match="not held"):
        m.ensure(s, 1)
    with pytest.raises(CacheError):
        CacheManager([FULL], page_size=0, max_total_tokens=16, max_slots=1)


def test_borrowed_cache_and_state_slots_and_no_cache():
    m = CacheManager([FULL, ("borrow", 0), StateNeed((3,)), None], page_size=4, max_total_tokens=16, max_slots=2)
    assert m.stage_group[1] == m.stage_group[0] and 2 in m.stage_state and 3 not in m.stage_group
    with pytest.raises(CacheError, match="borrows"):
        CacheManager([StateNeed((3,)), ("borrow", 0)], page_size=4, max_total_tokens=16, max_slots=2)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_duplicate_a_page(seed):
    rng = random.Random(seed)
    m = CacheManager([FULL, WIN, PagedNeed(1, 32, 5)], page_size=4, max_total_tokens=64, max_slots=5)
    live = {}                                  # slot -> length
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.free_slots:
            live[m.admit()] = 0
        elif op < 0.40 and live:
            s = rng.choice(sorted(live))
            m.release(s)
            del live[s]
        elif live:
            s = rng.choice(sorted(live))
            new = live[s] + rng.randint(1, 9)
            try:
                m.ensure(s, new)
            except OutOfPages:
                assert not m.can_hold([(s, new)])
            else:
                m.commit(s, new)
                live[s] = new
        m.check_invariants()
        for s, n in live.items():
            assert m.length(s) == n
            for g in m.groups:                 # every position a future query can see has a page
                lo = 0 if g.need.window is None else max(0, n - g.need.window + 1)
                for pos in range(lo, n):
                    assert g.first_held[s] <= pos // 4 < g.num_logical[s]
    for s in list(live):
        m.release(s)
    m.check_invariants()
    assert all(g.pool.free_count == g.pool.num_pages for g in m.groups)


def test_reserve_adds_up_a_step_one_request_at_a_time():
    """`reserve` answers for one more request on top of what a step has promised already, and
    agrees with `can_hold` for the whole list; it takes nothing itself."""
    m = CacheManager([FULL], page_size=4, max_total_tokens=24, max_slots=4, max_request_tokens=16)   # 6 pages
    a = m.admit()
    m.ensure(a, 6)
    m.commit(a, 6)                                           # holds 2 pages, 4 free
    need = m.reserve([0], a, 7)
    assert need == [0]                                       # position 6 lies in a page it has
    need = m.reserve(need, a, 9)
    assert need == [1]
    need2 = m.reserve(need, None, 9)                         # a newcomer of 9 tokens: 3 pages
    assert need2 == [4] and m.can_hold([(a, 9), (None, 9)])
    assert m.reserve(need2, None, 1) is None and not m.can_hold([(a, 9), (None, 9), (None, 1)])
    assert m.reserve([0], None, 17) is None                  # longer than a request may be
    assert m.groups[0].pool.free_count == 4                  # asking took nothing
    m.check_invariants()


def test_keys_and_values_of_different_widths_get_a_group_of_their_own():
    narrow = PagedNeed(2, 16, None, value_dim=8)
    assert (narrow.key_width, narrow.value_width) == (16, 8) and (FULL.key_width, FULL.value_width) == (16, 16)
    m = CacheManager([FULL, narrow, FULL, narrow], page_size=4, max_total_tokens=32, max_slots=2)
    assert [g.stages for g in m.groups] == [[0, 2], [1, 3]]
    assert m.bytes_per_token() == 2 * (2 * (16 + 16) + 2 * (16 + 8)) * 2          # two stages each, 2-byte elements
    s = m.admit()
    m.ensure(s, 9)
    assert [len(g.held_pages(s)) for g in m.groups] == [3, 3]
    m.release(s)
    m.check_invariants()
