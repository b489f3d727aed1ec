"""The cache manager: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; exhaustion takes nothing."""
import random

import pytest

from neurogrid_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagedNeed, PagePool


def mgr(pages=(16,), page_size=8, max_requests=4, max_seq_len=256, windows=(None,)):
    needs = [PagedNeed(2, 16, w) for w in windows]
    return CacheManager(needs, list(pages), page_size, max_requests, max_seq_len)


def test_pool_refuses_double_free_and_foreign_pages():
    p = PagePool(3)
    a = p.take(2)
    assert p.free == 1 and sorted(a) == [0, 1]
    p.give_back(a[0])
    with pytest.raises(RuntimeError):
        p.give_back(a[0])
    with pytest.raises(ValueError):
        p.give_back(7)
    with pytest.raises(OutOfPages):
        p.take(3)
    assert p.free == 2                                        # a refused request takes nothing


def test_pages_follow_tokens_and_are_reused():
    m = mgr()
    m.admit("a")
    m.extend("a", 5); m.advance("a", 5)
    assert m.pages_held("a") == [1]
    m.extend("a", 3); m.advance("a", 3)                       # fills the page exactly
    assert m.pages_held("a") == [1]
    m.extend("a", 1); m.advance("a", 1)
    assert m.pages_held("a") == [2] and m.length("a") == 9
    first = list(m.table("a", 0))
    m.release("a")
    assert m.pages_free() == [16]
    m.admit("b")
    m.extend("b", 9)
    assert set(m.table("b", 0)) == set(first)                 # LIFO: the same pages come back
    m.check()


def test_exhaustion_is_all_or_nothing_across_groups():
    m = mgr(pages=(4, 2), windows=(None, None))
    m.admit("a")
    m.extend("a", 16); m.advance("a", 16)                     # 2 pages in each group
    assert not m.can_extend("a", 8)
    with pytest.raises(OutOfPages):
        m.extend("a", 8)                                      # group 1 is full: group 0 must not be touched
    assert m.pages_free() == [2, 0] and m.pages_held("a") == [2, 2]
    m.check()


def test_capacity_and_slots():
    m = mgr(max_requests=2, max_seq_len=20)
    m.admit(1); m.admit(2)
    with pytest.raises(OutOfSlots):
        m.admit(3)
    with pytest.raises(KeyError):
        m.admit(1)
    with pytest.raises(OutOfPages):
        m.extend(1, 21)
    m.extend(1, 20)
    with pytest.raises(RuntimeError):
        m.advance(2, 1)                                       # advancing beyond the pages taken
    assert m.release(1) in (0, 1)
    m.check()


def test_window_gives_pages_back_once_passed():
    m = mgr(pages=(12, 6), page_size=4, windows=(None, 6), max_seq_len=64)
    m.admit("a")
    for _ in range(20):
        m.extend("a", 1); m.advance("a", 1)
        m.check()
    # 20 tokens: the full group holds 5 pages; the window group only those reaching back 6 keys
    assert m.pages_held("a") == [5, 2]
    t = m.table("a", 1)
    assert t[:3] == [-1, -1, -1] and all(p >= 0 for p in t[3:])
    # a long portion needs all its pages during the step, whatever the window
    m.admit("b")
    m.extend("b", 16); m.advance("b", 16)
    assert m.pages_held("b")[1] == 4
    m.extend("b", 1); m.advance("b", 1)
    assert m.pages_held("b")[1] == 3                          # keys 11..16 stay visible: pages 2, 3 and the new page 4
    m.release("a"); m.release("b")
    assert m.pages_free() == [12, 6]


def test_window_never_frees_a_visible_key():
    ps, w = 4, 5
    m = mgr(pages=(64,), page_size=ps, windows=(w,), max_seq_len=200)
    m.admit("a")
    rng = random.Random(1)
    while m.length("a") < 150:
        n = rng.choice([1, 1, 2, 7, 13])
        m.extend("a", n)
        first_query = m.length("a")
        t = m.table("a", 0)
        for key in range(max(0, first_query - w + 1), first_query + n):
            assert t[key // ps] >= 0, (first_query, n, key)
        m.advance("a", n)
        m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = mgr(pages=(24, 10), page_size=4, max_requests=5, windows=(None, 9), max_seq_len=80)
    live, nxt = [], 0
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and len(live) < 5:
            m.admit(nxt); live.append(nxt); nxt += 1
        elif op < 0.8 and live:
            r = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 5, 17])
            before = (m.pages_free(), m.pages_held(r), m.length(r))
            if m.can_extend(r, n):
                m.extend(r, n); m.advance(r, n)
            else:
                with pytest.raises(OutOfPages):
                    m.extend(r, n)
                assert before == (m.pages_free(), m.pages_held(r), m.length(r))
        elif live:
            r = live.pop(rng.randrange(len(live)))
            m.release(r)
        m.check()
    for r in live:
        m.release(r)
    m.check()
    assert m.pages_free() == [24, 10] and m.slots_free() == 5
