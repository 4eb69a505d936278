"""The cache manager: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; shortage changes nothing."""

import random

import numpy as np
import pytest

from yalis_b200.cache.manager import CacheError, CacheManager, PageGroup


def two_groups(pages=12, page=4, window=10, width=32, slots=4):
    return CacheManager(slots, [PageGroup("kv_all", page, pages, None, width),
                                PageGroup(f"kv_window_{window}", page, pages, window, width)])


def held_pages(m, group):
    t = m.table(group)
    return sorted(int(p) for p in t.ravel() if p >= 0)


def test_reserve_commit_release_basic():
    m = two_groups()
    s = m.acquire()
    assert s == 0 and m.acquire() == 1          # smallest free slot first
    assert m.reserve(s, 9)                      # 3 pages of 4 in each group
    assert list(m.table("kv_all")[s, :4]) == [0, 1, 2, -1]
    assert m.free_pages("kv_all") == 9 and m.free_pages("kv_window_10") == 9
    assert m.reserve(s, 9) and m.free_pages("kv_all") == 9      # idempotent
    assert m.commit(s, 9) == 0 and m.length(s) == 9
    m.check()
    assert m.release(s) == 6 and m.free_pages("kv_all") == 12
    assert m.acquire() == 0                     # the slot is reused, with length 0
    assert m.length(0) == 0
    m.check()


def test_pages_are_reused_most_recent_first():
    m = CacheManager(2, [PageGroup("kv_all", 4, 6, None, 6)])
    a, b = m.acquire(), m.acquire()
    m.reserve(a, 8); m.reserve(b, 8)
    first = list(m.table("kv_all")[a, :2])
    m.release(a)
    a2 = m.acquire()
    m.reserve(a2, 8)
    assert sorted(m.table("kv_all")[a2, :2]) == sorted(first)     # the freed pages come straight back
    m.check()


def test_window_group_gives_pages_back_at_commit():
    m = two_groups(pages=12, page=4, window=10)
    s = m.acquire()
    m.reserve(s, 30)
    m.commit(s, 30)
    # a query at position 30 sees keys 21..30: pages 5.. ; pages 0-4 of the window group are free again
    w = m.table("kv_window_10")[s]
    assert all(w[i] == -1 for i in range(5)) and all(w[i] >= 0 for i in range(5, 8))
    assert m.held_range("kv_window_10", s) == (5, 8)
    assert all(m.table("kv_all")[s][i] >= 0 for i in range(8))
    assert m.free_pages("kv_window_10") == 12 - 3 and m.free_pages("kv_all") == 12 - 8
    m.check()
    # growing by one page needs one page in each group, whatever was given back
    assert m.pages_needed(s, 34) == {"kv_all": 1, "kv_window_10": 1}


def test_window_never_drops_a_visible_key():
    page, window = 4, 6
    m = CacheManager(1, [PageGroup("w", page, 64, window, 64)])
    s = m.acquire()
    length = 0
    rng = random.Random(0)
    while length < 200:
        length += rng.choice([1, 1, 2, 5, 13])
        assert m.reserve(s, length)
        # every key a query of this step can see is mapped *during* the step
        m.commit(s, length)
        row = m.table("w")[s]
        for key in range(max(0, length - window + 1), length):
            assert row[key // page] >= 0, (length, key)
        # and nothing more than the window plus one page of slack stays held
        lo, hi = m.held_range("w", s)
        assert (hi - lo) * page <= window + 2 * page
        m.check()


def test_shortage_changes_nothing():
    m = CacheManager(2, [PageGroup("kv_all", 4, 5, None, 16)])
    a, b = m.acquire(), m.acquire()
    assert m.reserve(a, 12)                       # 3 of 5 pages
    before = m.table("kv_all").copy()
    assert not m.can_reserve(b, 12)
    assert m.reserve(b, 12) is False              # needs 3, 2 left
    assert np.array_equal(before, m.table("kv_all")) and m.free_pages("kv_all") == 2
    assert m.reserve(b, 8)                        # 2 pages do fit
    m.check()


def test_a_refused_step_leaves_every_page_where_it_was():
    """``reserve_many`` is for all requests of a step or for none: a step that does not fit takes no page from
    the requests named first, so a caller that retries with a smaller batch finds the pool unchanged."""
    m = two_groups(pages=6, page=4, window=10)
    a, b, c = m.acquire(), m.acquire(), m.acquire()
    assert m.reserve_many([a, b], [8, 4]) and m.free_pages("kv_all") == 3
    m.commit(a, 8); m.commit(b, 4)
    before = (m.free_pages("kv_all"), m.free_pages("kv_window_10"), m.table("kv_all").copy())
    assert not m.reserve_many([a, b, c], [12, 8, 8])          # needs 1 + 1 + 2 pages, 3 are free
    assert (m.free_pages("kv_all"), m.free_pages("kv_window_10")) == before[:2]
    assert np.array_equal(m.table("kv_all"), before[2])
    m.check()
    assert m.reserve_many([a, b], [12, 8]) and m.free_pages("kv_all") == 1      # the smaller step fits
    assert m.reserve_many([], [])
    with pytest.raises(CacheError):
        m.reserve_many([a, a], [13, 13])
    with pytest.raises(CacheError):
        m.reserve_many([a], [13, 14])
    with pytest.raises(CacheError):
        m.reserve_many([a], [4])                               # below what it holds
    m.check()


def test_commit_many_is_commit_for_every_request_of_a_step():
    """One call for all requests of a step: the same lengths, the same pages given back behind a window as
    request by request, and a wrong entry changes nothing for the others."""
    m, ref = two_groups(pages=24, page=4, window=10), two_groups(pages=24, page=4, window=10)
    slots = [m.acquire(), m.acquire(), m.acquire()]
    assert [ref.acquire() for _ in range(3)] == slots
    for lens in ([5, 9, 1], [17, 10, 2], [30, 11, 16]):
        assert m.reserve_many(slots, lens) and ref.reserve_many(slots, lens)
        given_back = m.commit_many(slots, lens)
        assert given_back == sum(ref.commit(s, n) for s, n in zip(slots, lens))
        assert [m.length(s) for s in slots] == lens
        for g in ("kv_all", "kv_window_10"):
            assert np.array_equal(m.table(g), ref.table(g)) and m.free_pages(g) == ref.free_pages(g)
        m.check()
    assert m.commit_many([], []) == 0
    with pytest.raises(CacheError):
        m.commit_many([slots[0], slots[1]], [31, 40])              # the second has no pages for 40 tokens
    assert m.length(slots[0]) == 30                                 # and the first was not touched
    with pytest.raises(CacheError):
        m.commit_many([slots[0]], [29])                             # shorter than what it holds
    m.check()


def test_groups_with_a_window_get_no_more_pages_than_they_can_use():
    from yalis_b200.cache.storage import group_page_bytes, plan_groups, window_group_pages
    from yalis_b200.parts.base import PagedKV, SlotState
    requests = [PagedKV(2, 16), PagedKV(2, 16, window=20), None, SlotState((5,)), PagedKV(4, 32)]
    groups = {g.name: g for g in plan_groups(requests, page_size=8, num_pages=1000, max_context=4096, max_slots=4, step_tokens=64)}
    assert groups["kv_all"].num_pages == 1000
    assert groups["kv_window_20"].num_pages == window_group_pages(20, 8, 4, 64) == 4 * (11 + 2)
    assert {g.name: g.num_pages for g in plan_groups(requests, 8, 1000, 4096)} == {"kv_all": 1000, "kv_window_20": 1000}
    assert group_page_bytes(requests, [None, None, None, None, 0], 8, 2) == {"kv_all": 2 * 2 * 8 * 16 * 2, "kv_window_20": 2 * 2 * 8 * 16 * 2}
    assert group_page_bytes(requests, [None] * 5, 8, 2)["kv_all"] == 2 * 2 * 8 * 16 * 2 + 2 * 4 * 8 * 32 * 2


def test_misuse_raises():
    m = two_groups()
    with pytest.raises(CacheError):
        m.release(0)                              # never acquired
    s = m.acquire()
    m.reserve(s, 8); m.commit(s, 8)
    with pytest.raises(CacheError):
        m.commit(s, 4)                            # lengths do not shrink
    with pytest.raises(CacheError):
        m.commit(s, 50)                           # beyond the reserved pages
    with pytest.raises(CacheError):
        m.reserve(s, 10 ** 6)                     # wider than a block-table row
    assert not m.fits(10 ** 6) and m.fits(100)
    m.release(s)
    with pytest.raises(CacheError):
        m.release(s)                              # freed twice
    with pytest.raises(CacheError):
        m.reserve(s, 4)                           # slot not in use
    with pytest.raises(ValueError):
        PageGroup("x", 0, 1, None, 1)
    with pytest.raises(ValueError):
        CacheManager(1, [PageGroup("x", 1, 1, None, 1), PageGroup("x", 1, 1, None, 1)])


@pytest.mark.parametrize("seed", range(6))
def test_random_lifetimes_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    page, pages, window = rng.choice([1, 4, 16]), rng.choice([7, 20, 64]), rng.choice([3, 17, 40])
    m = CacheManager(5, [PageGroup("kv_all", page, pages, None, 64), PageGroup("w", page, pages, window, 64)])
    live = {}                                     # slot -> committed length
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            s = m.acquire()
            assert s is not None and s not in live
            live[s] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            grow = rng.choice([1, 1, 1, 2, 7, 30])
            new_len = live[s] + grow
            if not m.fits(new_len):
                continue
            could = m.can_reserve(s, new_len)
            free_before = {g.name: m.free_pages(g.name) for g in m.groups}
            ok = m.reserve(s, new_len)
            assert ok == could
            if ok:
                m.commit(s, new_len)
                live[s] = new_len
            else:
                assert free_before == {g.name: m.free_pages(g.name) for g in m.groups}
        elif live:
            s = rng.choice(list(live))
            m.release(s)
            del live[s]
        m.check()                                  # no page lost, held twice or free twice
        assert m.free_slots() == 5 - len(live)
        for g in m.groups:
            held = held_pages(m, g.name)
            assert len(held) == len(set(held)) and len(held) + m.free_pages(g.name) == pages
        for s, n in live.items():
            assert m.length(s) == n
    for s in list(live):
        m.release(s)
    for g in m.groups:
        assert m.free_pages(g.name) == pages
