"""Page allocator and cache manager invariants (no GPU): no page lost, held twice or freed twice,
under random orders of requests.  After the reference's allocator and sequence tests
(tests/backend_tests.cpp:750-1084)."""
import random

import pytest

from mimirmind_b200.cache import CacheError, CacheManager, GroupSpec, INVALID_PAGE, PageAllocator, PageAllocatorError


def test_allocator_ascending_then_lifo_reuse():
    a = PageAllocator(4)
    assert [a.alloc() for _ in range(4)] == [0, 1, 2, 3]
    assert a.alloc() == INVALID_PAGE          # exhaustion is a sentinel, never an exception
    a.free(2)
    a.free(0)
    assert a.alloc() == 0 and a.alloc() == 2   # last freed, first reused
    assert a.reuses == 2
    a.check()


def test_allocator_double_free_and_foreign_page():
    a = PageAllocator(3)
    p = a.alloc()
    a.free(p)
    with pytest.raises(PageAllocatorError, match="twice"):
        a.free(p)
    with pytest.raises(PageAllocatorError, match="outside"):
        a.free(7)
    with pytest.raises(PageAllocatorError):
        a.free(1)                              # never allocated


def test_alloc_many_is_all_or_nothing():
    a = PageAllocator(3)
    assert a.alloc_many(4) is None and a.num_free == 3
    assert a.alloc_many(3) == [0, 1, 2]


def groups(window=0):
    g = [GroupSpec("full", (0, 2), 2, 16, 0)]
    if window:
        g.append(GroupSpec("win", (1,), 1, 32, window))
    return g


def test_reserve_commit_release():
    m = CacheManager(groups(), page_size=16, pages_per_group=4, max_requests=2)
    assert m.add_request("a") == 0
    assert m.reserve("a", 17)                  # two pages
    assert m.table("a", "full") == [0, 1]
    assert m.length("a") == 0                  # rows count only after commit
    m.commit("a", 17)
    assert m.length("a") == 17
    assert m.reserve("a", 32) and m.table("a", "full") == [0, 1]   # same page, no new one
    assert m.reserve("a", 33) and m.table("a", "full") == [0, 1, 2]
    m.check()
    m.release("a")
    assert m.free_pages() == 4
    m.check()


def test_reserve_is_all_or_nothing_across_groups():
    m = CacheManager(groups(window=8), page_size=4, pages_per_group={"full": 8, "win": 2}, max_requests=2)
    m.add_request("a")
    before = (m.free_pages("full"), m.free_pages("win"))
    assert not m.reserve("a", 12)              # the window group has only 2 pages, 3 are needed
    assert (m.free_pages("full"), m.free_pages("win")) == before
    assert m.table("a", "full") == []
    m.check()


def test_window_group_gives_pages_back_and_reuses_them():
    m = CacheManager(groups(window=8), page_size=4, pages_per_group={"full": 64, "win": 4}, max_requests=2)
    m.add_request("a")
    n = 0
    for step in range(40):                     # 3 tokens at a time, far beyond 4 pages of 4 tokens
        assert m.reserve("a", n + 3), f"step {step}"
        n += 3
        m.commit("a", n)
        m.check()
        t = m.table("a", "win")
        live = [i for i, p in enumerate(t) if p != INVALID_PAGE]
        # every position the next query can see still has its page
        for pos in range(max(0, n + 1 - 8), n):
            assert t[pos // 4] != INVALID_PAGE
        assert len(live) <= 4
    assert m.allocators["win"].reuses > 0
    assert all(p != INVALID_PAGE for p in m.table("a", "full"))   # the full group keeps everything


def test_state_slots_are_handed_back():
    m = CacheManager(groups(), 16, 8, max_requests=2)
    assert m.add_request("a") == 0 and m.add_request("b") == 1
    assert m.add_request("c") is None
    assert not m.has("c")
    m.release("a")
    assert m.add_request("c") == 0
    assert m.mark_started("c") and not m.mark_started("c")
    with pytest.raises(CacheError):
        m.add_request("c")
    with pytest.raises(CacheError):
        m.release("zzz")


def test_commit_bounds():
    m = CacheManager(groups(), 16, 8, 2)
    m.add_request("a")
    m.reserve("a", 10)
    with pytest.raises(CacheError):
        m.commit("a", 11)
    m.commit("a", 10)
    with pytest.raises(CacheError):
        m.commit("a", 5)
    with pytest.raises(CacheError):
        m.reserve("a", 5)


@pytest.mark.parametrize("seed", range(8))
def test_random_traces_keep_every_invariant(seed):
    rng = random.Random(seed)
    ps = rng.choice([4, 8, 16])
    m = CacheManager(groups(window=rng.choice([0, 12, 40])), ps, pages_per_group=rng.randint(6, 20), max_requests=4)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and len(live) < 4:
            rid = f"r{next_id}"
            next_id += 1
            assert m.add_request(rid) is not None
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            new_len = live[rid] + rng.randint(1, 3 * ps)
            free_before = {g: m.free_pages(g) for g in m.groups}
            if m.reserve(rid, new_len):
                if rng.random() < 0.9:
                    m.commit(rid, new_len)
                    live[rid] = new_len
            else:
                assert {g: m.free_pages(g) for g in m.groups} == free_before
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.length(rid) == n
    for rid in list(live):
        m.release(rid)
    m.check()
    for g in m.groups:
        assert m.free_pages(g) == m.total_pages(g)
