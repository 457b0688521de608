"""The cache's bookkeeping: no page or slot lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from pytorch_transformers_b200.cache import Cache, CacheError, CacheFull, IdPool, PAGE
from pytorch_transformers_b200.parts import CacheNeed, StateNeed


def make(max_tokens=64 * 8, window=0, state=0, max_slots=None):
    need = CacheNeed("window" if window else "full", 2, 4, window)
    return Cache([(0, need, StateNeed(state) if state else None), (1, need, None)], max_tokens, torch.float32, "cpu",
                 max_slots=max_slots)


def test_id_pool():
    p = IdPool(4, "page")
    a = p.take(3)
    assert a == [0, 1, 2] and p.available == 1 and p.in_use == 3
    with pytest.raises(CacheFull):
        p.take(2)
    p.give_back([1])
    with pytest.raises(CacheError, match="freed twice"):
        p.give_back([1])
    with pytest.raises(CacheError, match="outside"):
        p.give_back([9])
    with pytest.raises(CacheError, match="twice in one release"):
        p.give_back([0, 0])
    assert p.take(2) == [1, 3]
    p.check()


def test_sizes_and_groups():
    c = make(max_tokens=100)
    assert c.num_pages == 2 and c.max_tokens == 128          # rounded up to whole pages
    assert len(c.groups) == 1 and c.groups[0].k.shape == (2, 2, 2, PAGE, 4)
    two = Cache([(0, CacheNeed("full", 2, 4), None), (1, CacheNeed("window", 2, 4, 10), None),
                 (2, CacheNeed("full", 1, 8), None)], 640, torch.float32, "cpu")
    assert len(two.groups) == 3                              # different needs: storage of their own
    k, v, gi = two.entry_storage(1)
    assert two.groups[gi].need.kind == "window" and k.shape == (10, 2, PAGE, 4)
    assert c.state.shape == (c.max_slots, 0)                 # the state area exists, empty


def test_open_reserve_commit_close():
    c = make()
    s = c.open()
    assert c.length(s) == 0
    c.reserve(s, 65)
    assert len(c.pages(s, 0)) == 2
    c.commit(s, 65)
    c.reserve(s, 1)
    assert len(c.pages(s, 0)) == 2
    c.commit(s, 1)
    with pytest.raises(CacheError, match="beyond its reserved pages"):
        c.commit(s, 200)
    c.close(s)
    with pytest.raises(CacheError, match="not open"):
        c.close(s)
    with pytest.raises(CacheError, match="not open"):
        c.length(s)
    c.check()
    assert c.groups[0].pool.in_use == 0


def test_full_cache_raises_before_anything_is_kept():
    c = make(max_tokens=64 * 4)
    a, b = c.open(), c.open()
    c.reserve_all([(a, 64), (b, 64)])
    c.commit(a, 64)
    c.commit(b, 64)
    with pytest.raises(CacheFull, match="sized for 256 tokens"):
        c.reserve_all([(a, 64), (b, 65)])      # would need 3 more pages, 2 are free
    assert len(c.pages(a, 0)) == 1 and len(c.pages(b, 0)) == 1
    c.check()


def test_slots_are_used_again_lowest_first():
    c = make(max_slots=3)
    s = [c.open() for _ in range(3)]
    assert s == [0, 1, 2]
    with pytest.raises(CacheFull, match="sequence slot"):
        c.open()
    c.close(1)
    assert c.open() == 1


def test_window_group_gives_pages_back():
    c = make(max_tokens=64 * 4, window=70)
    s = c.open()
    held = []
    for _ in range(20):                       # 20 * 50 = 1000 tokens through a 256-token cache
        c.reserve(s, 50)
        c.commit(s, 50)
        held.append(sum(1 for p in c.pages(s, 0) if p >= 0))
        c.check()
    assert max(held) <= 3 and c.length(s) == 1000
    # the pages still held cover every position a later query may see
    first_needed = 1000 - 70 + 1
    assert all(p >= 0 for p in c.pages(s, 0)[first_needed // PAGE:])
    c.close(s)
    assert c.groups[0].pool.in_use == 0


def test_state_area_is_zeroed_for_a_new_sequence():
    c = make(state=5)
    s = c.open()
    st = c.entry_state(0)
    assert st.shape == (c.max_slots, 5) and c.entry_state(1) is None
    st[s] += 3.0
    c.close(s)
    s2 = c.open()
    assert s2 == s and torch.all(c.entry_state(0)[s2] == 0)


def test_random_traffic_keeps_the_invariants():
    rng = random.Random(0)
    c = make(max_tokens=64 * 16, max_slots=6)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and len(live) < 6:
            live[c.open()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 7, 64, 100])
            try:
                c.reserve_all([(s, n)])
                c.commit(s, n)
                live[s] += n
            except CacheFull:
                pass
        elif live:
            s = rng.choice(list(live))
            c.close(s)
            del live[s]
        c.check()
        assert c.live_tokens() == sum(live.values())
        assert c.groups[0].pool.in_use >= sum((n + PAGE - 1) // PAGE for n in live.values())
    c.close_all()
    c.check()
    assert c.groups[0].pool.in_use == 0 and c.slots.in_use == 0


def test_another_cache_kind_is_registered_not_edited_in():
    """A kind of cache entry is a rule that says which positions later queries may still read; pages
    wholly before them go back to the pool after every step. Here: chunks of 128 tokens, a query reads
    its own chunk only."""
    from pytorch_transformers_b200.cache.paged import CACHE_KINDS, register_cache_kind
    register_cache_kind("chunk128", lambda need, length: length // 128 * 128)
    try:
        cache = Cache([(0, CacheNeed("chunk128", 1, 16), None), (1, CacheNeed("full", 1, 16), None)], 64 * 16,
                      torch.float32, "cpu")
        chunked = next(i for i, g in enumerate(cache.groups) if g.need.kind == "chunk128")
        full = 1 - chunked
        s = cache.open()
        for n in (100, 100, 100):
            cache.reserve(s, n)
            cache.commit(s, n)
        # 300 tokens: the chunk in use starts at 256; the pages of positions 0..255 are back in the pool
        assert cache.pages(s, chunked)[:4] == [-1] * 4 and all(p >= 0 for p in cache.pages(s, chunked)[4:])
        assert all(p >= 0 for p in cache.pages(s, full)) and len(cache.pages(s, full)) == 5
        assert cache.groups[chunked].pool.in_use == 1 and cache.groups[full].pool.in_use == 5
        cache.check()
        cache.close(s)
        assert cache.groups[chunked].pool.in_use == 0
        with pytest.raises(ValueError, match="unknown cache kind"):
            Cache([(0, CacheNeed("ring", 1, 16), None)], 64, torch.float32, "cpu")
    finally:
        del CACHE_KINDS["chunk128"]
