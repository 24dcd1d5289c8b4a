"""The cache manager on the CPU: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; reuse."""
import random

import pytest

from tuff_b200.cache import NO_PAGE, CacheManager, OutOfPages, PoolError, UnitPool
from tuff_b200.parts import PagedKVNeed, StateNeed


def needs(window=None):
    return [StateNeed((2, 8)), PagedKVNeed(2, 16), PagedKVNeed(2, 16), None, PagedKVNeed(1, 24, window=window)]


def test_pool_rules():
    p = UnitPool(3)
    a = p.take(2)
    assert a == [0, 1] and p.n_free == 1
    with pytest.raises(OutOfPages):
        p.take(2)
    assert p.n_free == 1                      # a refused request takes nothing
    p.give_back(0)
    with pytest.raises(PoolError):
        p.give_back(0)                        # freed twice
    with pytest.raises(PoolError):
        p.give_back(2)                        # never taken
    with pytest.raises(PoolError):
        p.give_back(7)                        # not of this pool
    assert p.take(1) == [0]                   # the page freed last is used again first
    p.check()


def test_groups_by_need():
    cm = CacheManager(needs(window=8), page_size=4, max_tokens=64, max_requests=3)
    assert len(cm.groups) == 2                # all-keys layers share a group, the windowed layer has its own
    assert cm.groups[0].storages == [1, 2] and cm.groups[1].storages == [4]
    assert cm.storages[3] is None and cm.storages[0].shape == (2, 8)
    assert cm.num_pages == 16


def test_reserve_commit_close_and_reuse():
    cm = CacheManager(needs(), page_size=4, max_tokens=32, max_requests=2)     # 8 pages per group
    a = cm.open("a")
    cm.reserve(a, 9)
    assert [len(t) for t in a.tables] == [3, 3]
    cm.commit(a, 9)
    cm.reserve(a, 3)                          # positions 9..11 still fit block 2
    assert [len(t) for t in a.tables] == [3, 3]
    cm.commit(a, 3)
    cm.reserve(a, 1)
    assert len(a.tables[0]) == 4
    cm.cancel(a)                              # the step did not run: the fourth page goes back
    assert len(a.tables[0]) == 3 and a.n_tokens == 12
    b = cm.open("b")
    with pytest.raises(OutOfPages):
        cm.reserve(b, 21)                     # 6 pages wanted, 5 free
    assert b.tables == [[], []] and cm.groups[0].pool.n_free == 5
    with pytest.raises(PoolError):
        cm.open("a")
    with pytest.raises(OutOfPages):
        cm.open("c")                          # no slot left
    old = list(a.tables[0])
    cm.close(a)
    with pytest.raises(PoolError):
        cm.close(a)
    c = cm.open("c")
    cm.reserve(c, 12)
    assert sorted(c.tables[0]) == sorted(old)  # a's pages serve c
    cm.check()


def test_window_gives_pages_back():
    cm = CacheManager(needs(window=6), page_size=4, max_tokens=64, max_requests=2)
    a = cm.open("a")
    held = []
    for _ in range(40):
        cm.reserve(a, 1)
        cm.commit(a, 1)
        live = [p for p in a.tables[1] if p != NO_PAGE]
        held.append(len(live))
        first_needed = a.n_tokens - 6 + 1
        for b, p in enumerate(a.tables[1]):   # a block is gone exactly when the window has passed all of it
            assert (p == NO_PAGE) == ((b + 1) * 4 <= first_needed)
    assert max(held) <= 3                     # window 6 with pages of 4 never needs more than 3 pages
    assert len([p for p in a.tables[0] if p != NO_PAGE]) == 10   # the all-keys group keeps everything
    cm.check()
    cm.close(a)
    assert cm.groups[0].pool.n_free == cm.groups[1].pool.n_free == 16


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_invariants(seed):
    rng = random.Random(seed)
    cm = CacheManager(needs(window=rng.choice([None, 5, 16])), page_size=rng.choice([1, 2, 4, 16]),
                      max_tokens=96, max_requests=4)
    live, n_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and cm.can_open():
            live[n_id] = cm.open(n_id)
            n_id += 1
        elif op < 0.75 and live:
            rc = rng.choice(list(live.values()))
            n = rng.choice([1, 1, 1, 2, 3, 7, 20])
            before = [list(t) for t in rc.tables]
            try:
                cm.reserve(rc, n)
            except OutOfPages:
                assert [list(t) for t in rc.tables] == before
            else:
                if rng.random() < 0.15:
                    cm.cancel(rc)
                else:
                    cm.commit(rc, n)
        elif live:
            k = rng.choice(list(live))
            cm.close(live.pop(k))
        cm.check()
        # what a reader needs is there: every block from the window's start to the end has a page
        for rc in live.values():
            for g, table in zip(cm.groups, rc.tables):
                lo = 0 if g.need.window is None else max(0, rc.n_tokens - g.need.window + 1)
                for b in range(lo // cm.page_size, (rc.n_tokens + cm.page_size - 1) // cm.page_size):
                    assert table[b] != NO_PAGE
    for rc in list(live.values()):
        cm.close(rc)
    cm.check()
    assert all(g.pool.n_free == g.pool.n_units for g in cm.groups) and cm.slots.n_free == 4


def test_block_table_array():
    cm = CacheManager(needs(), page_size=4, max_tokens=64, max_requests=3)
    a, b = cm.open("a"), cm.open("b")
    cm.reserve(a, 10); cm.reserve(b, 3)
    t = cm.block_table(0, [b, a])
    assert t.shape == (2, 3) and t.dtype.name == "int32"
    assert list(t[0]) == [b.tables[0][0], NO_PAGE, NO_PAGE] and list(t[1]) == a.tables[0]
