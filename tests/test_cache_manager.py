"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; exhaustion is all-or-nothing.  Every test of the
manager runs on the C++ host runtime and on its Python twin."""
import random

import pytest

from host_twin import TwinCacheManager as CacheManager, PagePool, SlotPool
from tffinfer_b200.cache import (NativeCacheManager, GroupSpec, CacheAccountingError,
                                 NO_PAGE)


@pytest.fixture(params=[NativeCacheManager, CacheManager], ids=["native", "python"])
def Manager(request):
    return request.param


def test_pool_lifo_and_double_free():
    p = PagePool(4)
    a = p.alloc(3, "x")
    assert a == [0, 1, 2] and p.num_free == 1
    assert p.alloc(2, "y") is None and p.num_free == 1          # nothing taken
    p.free([1], "x")
    assert p.alloc(1, "y") == [1]                               # last freed, first reused
    with pytest.raises(CacheAccountingError, match="owned by"):
        p.free([0], "y")
    p.free([0, 2], "x")
    with pytest.raises(CacheAccountingError, match="twice"):
        p.free([0], "x")
    p.check()


def test_slots():
    s = SlotPool(2)
    a, b = s.alloc("a"), s.alloc("b")
    assert {a, b} == {0, 1} and s.alloc("c") is None
    s.free(a, "a")
    with pytest.raises(CacheAccountingError):
        s.free(a, "a")
    assert s.alloc("c") == a
    s.check()


def _mgr(Manager, pages=8, page=4, groups=None, live=4):
    groups = groups or [GroupSpec(2, 2, 16, 0)]
    return Manager(groups, page, [pages] * len(groups), live)


def test_reserve_is_all_or_nothing_across_groups(Manager):
    m = Manager([GroupSpec(2, 2, 16, 0), GroupSpec(1, 2, 16, 8)], 4, [8, 2], 4)
    assert m.admit("a") == 0
    assert m.reserve("a", 8)            # 2 pages in each group
    m.commit("a", 8)
    assert m.admit("b") is not None
    free_before = [p.num_free for p in m.pools]
    assert not m.reserve("b", 9)        # group 1 has no page left for b (a's window still needs both)
    assert [p.num_free for p in m.pools] == free_before
    m.check()
    m.release("a")
    assert m.reserve("b", 8)
    m.check()


def test_growth_page_by_page_and_block_table(Manager):
    m = _mgr(Manager)
    m.admit("a")
    for n in range(1, 14):
        assert m.reserve("a", 1)
        m.commit("a", 1)
        assert len(m.block_table("a", 0)) == -(-n // 4)
    assert m.num_tokens("a") == 13
    with pytest.raises(CacheAccountingError, match="reserved"):
        m.commit("a", 4)                # 13 + 4 > 16 reserved
    m.release("a")
    assert m.pools[0].num_free == 8
    m.check()


def test_window_gives_pages_back_when_passed(Manager):
    m = Manager([GroupSpec(1, 1, 16, 0), GroupSpec(1, 1, 16, 6)], 4, [16, 16], 2)
    m.admit("a")
    assert m.reserve("a", 20)
    m.commit("a", 20)
    full, win = m.block_table("a", 0), m.block_table("a", 1)
    assert all(p != NO_PAGE for p in full) and len(full) == 5
    # next query is at position 20 and sees keys 15..20: blocks 0..2 (keys 0..11) are passed
    assert [p == NO_PAGE for p in win] == [True, True, True, False, False]
    assert m.pools[1].num_used == 2 and m.pools[0].num_used == 5
    # the freed pages are used again by the same request
    assert m.reserve("a", 12)
    m.commit("a", 12)
    assert m.pools[1].num_used <= 3
    m.check()
    m.release("a")
    assert m.pools[1].num_free == 16
    m.check()


def test_random_orders_never_lose_or_double_book_a_page(Manager):
    rng = random.Random(11)
    m = Manager([GroupSpec(3, 2, 16, 0), GroupSpec(2, 2, 16, 10)], 4, [24, 12], 5)
    live, next_id, refused = {}, 0, 0
    for _ in range(3000):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            r = f"r{next_id}"; next_id += 1
            if m.admit(r) is not None:
                live[r] = 0
            else:
                assert len(live) == 5
        elif op < 0.85 and live:
            r = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 5, 9, 17])
            before = [p.num_free for p in m.pools]
            if m.reserve(r, n):
                k = rng.randint(0, n)            # a step may write fewer tokens than it reserved
                m.commit(r, k)
                live[r] += k
            else:
                refused += 1
                assert [p.num_free for p in m.pools] == before
        elif live:
            r = rng.choice(sorted(live))
            m.release(r)
            del live[r]
        m.check()
        for r, n in live.items():
            assert m.num_tokens(r) == n
    assert refused > 0
    for r in list(live):
        m.release(r)
    m.check()
    assert all(p.num_free == p.num_pages for p in m.pools) and m.slots.num_free == 5


def test_misuse_is_an_error_not_a_wrong_result(Manager):
    m = _mgr(Manager, live=2)
    assert m.admit("a") == 0
    with pytest.raises(CacheAccountingError, match="already live"):
        m.admit("a")
    with pytest.raises(KeyError):
        m.num_tokens("nobody")
    with pytest.raises(KeyError):
        m.reserve("nobody", 1)
    with pytest.raises(ValueError):
        m.reserve("a", -1)
    assert m.reserve("a", 3)
    with pytest.raises(CacheAccountingError, match="reserved"):
        m.commit("a", 5)
    assert m.admit("b") == 1 and m.admit("c") is None          # no slot left: nothing taken
    assert not m.is_live("c")
    m.release("a")
    with pytest.raises(KeyError):
        m.release("a")
    m.check()
    assert m.stats()["live_requests"] == 1 and m.pools[0].num_free == 8
