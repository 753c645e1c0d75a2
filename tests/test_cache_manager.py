"""The cache manager: pages, block tables, groups, windows, state slots (CPU)."""

import random

import pytest

from tandem_b200.cache.manager import CacheManager, KVNeed
from tandem_b200.cache.pages import OutOfPages, PagePool, SlotPool


def test_pool_fifo_reuse_and_double_free():
    pool = PagePool(4)
    a = pool.allocate(3)
    assert a == [0, 1, 2] and pool.num_free == 1
    pool.release([1])
    assert pool.allocate(2) == [3, 1]  # first freed, first reused (block_allocator.py:22,49 of the reference)
    with pytest.raises(OutOfPages):
        pool.allocate(1)
    pool.release([0])
    with pytest.raises(RuntimeError):
        pool.release([0])
    pool.share([2])
    pool.release([2])
    assert pool.holders(2) == 1 and pool.num_free == 1
    with pytest.raises(RuntimeError):
        pool.share([0])


def test_slot_pool():
    s = SlotPool(2)
    assert (s.acquire(), s.acquire()) == (0, 1)
    with pytest.raises(OutOfPages):
        s.acquire()
    s.release(0)
    with pytest.raises(RuntimeError):
        s.release(0)
    assert s.acquire() == 0


def test_groups_by_need():
    needs = [KVNeed(2, 16), KVNeed(2, 16, window=8), None, KVNeed(2, 16), KVNeed(4, 16), KVNeed(2, 16, window=8)]
    m = CacheManager(needs, page_size=4, num_pages=10, max_requests=3)
    assert [g.runs for g in m.groups] == [[0, 3], [1, 5], [4]]
    assert m.group_of_run == {0: 0, 3: 0, 1: 1, 5: 1, 4: 2}


def test_grow_is_all_or_nothing_and_end_gives_back():
    m = CacheManager([KVNeed(2, 16), KVNeed(1, 8)], page_size=4, num_pages=5, max_requests=4)
    m.begin("a")
    assert m.grow("a", 9)  # 3 pages in both groups
    m.commit("a", 9)
    m.begin("b")
    assert not m.grow("b", 12)  # would need 3, only 2 free
    assert m.table(0, "b") == [] and m.free_pages(0) == 2 and m.free_pages(1) == 2
    assert m.pages_short("b", 12) == 2 and m.pages_short("b", 8) == 0
    assert m.grow("b", 8)
    m.check()
    assert m.slot_index(0, "a", 6) == m.table(0, "a")[1] * 4 + 2
    m.end("a")
    m.end("b")
    assert m.all_free()
    with pytest.raises(KeyError):
        m.end("a")
    with pytest.raises(ValueError):
        m.begin("c") or m.begin("c")


def test_commit_beyond_pages_is_an_error():
    m = CacheManager([KVNeed(1, 8)], page_size=4, num_pages=4, max_requests=1)
    m.begin("a")
    m.grow("a", 4)
    with pytest.raises(RuntimeError):
        m.commit("a", 5)


def test_window_pages_come_back_when_passed():
    m = CacheManager([KVNeed(1, 8), KVNeed(1, 8, window=6)], page_size=4, num_pages=8, max_requests=2)
    m.begin("a")
    stored = 0
    for n in (5, 2, 9, 1, 1, 1, 6):
        assert m.grow("a", stored + n)
        m.commit("a", n)
        stored += n
        full, win = m.table(0, "a"), m.table(1, "a")
        assert all(p >= 0 for p in full) and len(full) == len(win) == -(-stored // 4)
        m.check()
    # the next query sits at position 25 and reads keys 20..25: pages 0..4 are passed once grow runs
    m.grow("a", stored + 1)
    assert [p >= 0 for p in m.table(1, "a")] == [False] * 5 + [True, True]
    with pytest.raises(RuntimeError):
        m.slot_index(1, "a", 3)
    assert m.free_pages(0) == 8 - 7 and m.free_pages(1) == 8 - 2
    m.end("a")
    assert m.all_free()


def test_window_lets_a_long_request_live_in_few_pages():
    m = CacheManager([KVNeed(1, 8, window=8)], page_size=4, num_pages=4, max_requests=1)
    m.begin("a")
    for t in range(200):  # token by token, far beyond 4 pages * 4 tokens
        assert m.grow("a", t + 1), t
        m.commit("a", 1)
    m.end("a")
    assert m.all_free()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    needs = [KVNeed(2, 16), KVNeed(2, 16, window=rng.choice([5, 9, 16])), KVNeed(1, 32)]
    m = CacheManager(needs, page_size=rng.choice([2, 4, 8]), num_pages=rng.choice([6, 11, 17]), max_requests=4)
    live, counter = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{counter}"
            counter += 1
            m.begin(rid)
            live[rid] = 0
        elif op < 0.85 and live:
            rid = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 13])
            before = [list(m.table(g, rid)) for g in range(len(m.groups))]
            free_before = [m.free_pages(g) for g in range(len(m.groups))]
            if m.grow(rid, live[rid] + n):
                m.commit(rid, n)
                live[rid] += n
            else:  # nothing taken (pages passed by a window may still have been given back)
                for g in range(len(m.groups)):
                    assert len(m.table(g, rid)) == len(before[g]) and m.free_pages(g) >= free_before[g]
        elif live:
            rid = rng.choice(sorted(live))
            m.end(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.num_tokens(rid) == n
    for rid in list(live):
        m.end(rid)
    assert m.all_free()
