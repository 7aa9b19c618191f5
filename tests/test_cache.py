import random

import pytest

from lumenllm_b200.cache import (PAGE, CacheError, CacheFull, CacheNeed, KVCache, PagePool,
                                 SlotAllocator, pages_for)


def test_slot_allocator_never_loses_or_doubles():
    a = SlotAllocator(4)
    got = [a.alloc() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        a.alloc()
    a.free(got[1])
    with pytest.raises(CacheError, match="freed twice"):
        a.free(got[1])
    with pytest.raises(CacheError, match="does not exist"):
        a.free(17)
    assert a.alloc() == got[1]          # what was given back last is used again first
    a.check()
    rng = random.Random(0)
    held = set(a.held)
    for _ in range(500):
        if held and rng.random() < 0.5:
            s = rng.choice(sorted(held))
            a.free(s)
            held.remove(s)
        elif len(held) < 4:
            s = a.alloc()
            assert s not in held
            held.add(s)
        a.check()
        assert a.held == held


def test_page_pool_reserves_page_zero_and_is_atomic():
    p = PagePool(5)
    assert p.capacity == 5
    with pytest.raises(CacheFull):
        p.take(6)
    assert p.free_count == 5            # a refused request takes nothing
    got = p.take(5)
    assert 0 not in got and sorted(got) == [1, 2, 3, 4, 5]
    with pytest.raises(CacheError):
        p.give_back([got[0], got[0]])
    p.give_back(got)
    p.check()


def _cache(window=0, max_tokens=640, slots=4):
    needs = {0: CacheNeed(2, 16, 0), 1: CacheNeed(2, 16, window), 2: CacheNeed(2, 16, 0)}
    return KVCache(needs, max_tokens, slots, max_positions=4096)


def test_groups_by_need():
    c = _cache(window=24)
    assert len(c.groups) == 2
    assert c.groups[c.group_of[0]].entries == [0, 2]
    assert c.groups[c.group_of[1]].entries == [1]
    same = _cache(window=0)
    assert len(same.groups) == 1


def test_lengths_pages_and_reuse():
    c = _cache()
    s = c.alloc_slot()
    assert c.reserve(s, 70) == 0
    g = c.groups[0]
    assert g.n_held[s] == pages_for(70) == 2
    c.commit(s, 70)
    assert c.length(s) == 70
    assert c.reserve(s, 1) == 70 and g.n_held[s] == 2     # position 70 is on page 1
    c.commit(s, 1)
    c.reserve(s, 58)
    assert g.n_held[s] == 3
    pages = g.table[s, :3].tolist()
    assert 0 not in pages and len(set(pages)) == 3
    c.check()
    c.free_slot(s)
    assert g.pool.free_count == g.pool.capacity
    with pytest.raises(CacheError):
        c.free_slot(s)
    with pytest.raises(CacheError, match="not live"):
        c.length(s)
    s2 = c.alloc_slot()
    assert s2 == s and c.length(s2) == 0
    c.reserve(s2, 10)
    assert g.table[s2, 0] == pages[-1] or g.table[s2, 0] in pages   # pages are used again
    c.check()


def test_full_cache_names_the_slot_and_keeps_state():
    c = _cache(max_tokens=128, slots=3)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve(a, 64); c.commit(a, 64)
    c.reserve(b, 64); c.commit(b, 64)
    with pytest.raises(CacheFull, match=f"slot {a}"):
        c.reserve(a, 1)
    assert c.length(a) == 64
    c.free_slot(b)
    c.reserve(a, 1)
    c.check()
    c.alloc_slot()
    c.alloc_slot()
    with pytest.raises(CacheFull):
        c.alloc_slot()


def test_window_group_gives_pages_back():
    c = _cache(window=24, max_tokens=64 * 8)
    s = c.alloc_slot()
    c.reserve(s, 200); c.commit(s, 200)
    gw = c.groups[c.group_of[1]]
    gf = c.groups[c.group_of[0]]
    assert gf.n_held[s] == 4
    # the next query sits at 200 and sees keys 177..200: pages 2 and 3
    assert gw.first_page[s] == 2 and gw.n_held[s] == 2
    for _ in range(60):
        c.reserve(s, 1); c.commit(s, 1)
    assert c.length(s) == 260
    assert gw.first_page[s] == (260 - 24 + 1) // PAGE == 3
    assert gf.n_held[s] == 5
    c.check()
    c.free_slot(s)
    assert gw.pool.free_count == gw.pool.capacity
    c.check()


def test_random_lifetimes_keep_the_books():
    rng = random.Random(1)
    c = _cache(window=24, max_tokens=64 * 40, slots=6)
    live = {}
    for _ in range(400):
        r = rng.random()
        if live and r < 0.2:
            s = rng.choice(sorted(live))
            c.free_slot(s)
            del live[s]
        elif len(live) < 6 and r < 0.45:
            s = c.alloc_slot()
            assert s not in live
            live[s] = 0
        elif live:
            s = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 5, 64, 100])
            try:
                c.reserve(s, n)
                c.commit(s, n)
                live[s] += n
            except CacheFull:
                pass
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
    for g in c.groups:
        pages = [p for s in live for p in g.table[s, int(g.first_page[s]):int(g.first_page[s] + g.n_held[s])].tolist()]
        assert len(pages) == len(set(pages)) and 0 not in pages     # no page held twice
