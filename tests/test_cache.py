import random

import pytest

from fieldrun_b200.cache import CacheFull, CacheNeed, IndexPool, PAGE_TOKENS, SequenceCache, pages_for


def test_pool_gives_each_index_once_and_reuses_freed_ones():
    pool = IndexPool(4, "slot")
    got = [pool.alloc() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        pool.alloc()
    pool.free(2)
    pool.free(0)
    assert pool.alloc() == 0 and pool.alloc() == 2
    pool.check()


def test_pool_refuses_double_free_and_strangers():
    pool = IndexPool(3, "page")
    a = pool.alloc()
    pool.free(a)
    with pytest.raises(ValueError, match="freed twice"):
        pool.free(a)
    with pytest.raises(ValueError, match="does not exist"):
        pool.free(7)
    with pytest.raises(ValueError, match="freed twice"):
        pool.free(2)           # never given out
    pool.check()


def _cache(max_tokens=640, slots=4, window=None, state=()):
    needs = [CacheNeed(2, 16, None), CacheNeed(2, 16, None), CacheNeed(2, 16, window) if window else CacheNeed(2, 16, None),
             CacheNeed(state_shape=state)]
    return SequenceCache(needs, max_tokens=max_tokens, num_slots=slots, device="cpu", allocate=bool(state))


def test_pages_follow_lengths_and_come_back():
    cache = _cache()
    a, b = cache.alloc(), cache.alloc()
    cache.begin_step([a, b], [5, 130])
    cache.end_step([a, b], [5, 130])
    assert cache.length(a) == 5 and cache.length(b) == 130
    group = cache.groups[0]
    assert group.pool.num_held == 1 + 3 and cache.tokens_held == 4 * PAGE_TOKENS
    for _ in range(59):
        cache.begin_step([a], [1]); cache.end_step([a], [1])
    assert cache.length(a) == 64 and group.pool.num_held == 4
    cache.begin_step([a], [1]); cache.end_step([a], [1])
    assert group.pool.num_held == 5
    cache.check()
    cache.free(b)
    assert group.pool.num_held == 2
    c = cache.alloc()
    assert c == b and cache.length(c) == 0                       # the slot is used again, empty
    cache.check()
    with pytest.raises(ValueError, match="freed twice"):
        cache.free(3)
    cache.free(a); cache.free(c)
    assert group.pool.num_held == 0 and cache.slots.num_held == 0
    cache.check()


def test_a_step_that_does_not_fit_changes_nothing():
    cache = _cache(max_tokens=256, slots=3)
    a, b = cache.alloc(), cache.alloc()
    cache.begin_step([a], [100]); cache.end_step([a], [100])
    held = cache.groups[0].pool.num_held
    with pytest.raises(CacheFull, match="pages"):
        cache.begin_step([a, b], [10, 200])
    assert cache.groups[0].pool.num_held == held and cache.length(b) == 0
    cache.check()
    with pytest.raises(ValueError, match="twice in one step"):
        cache.begin_step([a, a], [1, 1])
    with pytest.raises(ValueError, match="not held"):
        cache.begin_step([2], [1])


def test_groups_by_need_and_window_gives_pages_back():
    cache = _cache(max_tokens=1024, slots=2, window=100)
    assert len(cache.groups) == 2
    full = next(g for g in cache.groups if g.window is None)
    windowed = next(g for g in cache.groups if g.window == 100)
    assert full.lines == [0, 1] and windowed.lines == [2]
    s = cache.alloc()
    cache.begin_step([s], [300]); cache.end_step([s], [300])
    assert full.pool.num_held == pages_for(300)
    # the next query (position 300) sees keys 201..300: pages before 201 // 64 = 3 are given back
    assert windowed.pool.num_held == pages_for(300) - 3
    assert (windowed.table[s, :3] == -1).all() and windowed.table[s, 3] >= 0
    for _ in range(100):
        cache.begin_step([s], [1]); cache.end_step([s], [1])
    assert windowed.pool.num_held <= 3 and full.pool.num_held == pages_for(400)
    cache.check()
    cache.free(s)
    assert windowed.pool.num_held == 0 and full.pool.num_held == 0
    cache.check()


def test_state_is_zeroed_when_a_slot_is_given_out():
    cache = _cache(state=(3, 2))
    s = cache.alloc()
    view = cache.line(3)
    assert view.keys is None and view.state.shape == (4, 3, 2)
    view.state[s] += 5.0
    cache.free(s)
    assert cache.alloc() == s and float(cache.line(3).state[s].abs().sum()) == 0.0


def test_random_traffic_loses_nothing():
    rng = random.Random(0)
    cache = _cache(max_tokens=64 * 40, slots=6, window=70)
    live = {}
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and cache.slots.num_free:
            s = cache.alloc()
            live[s] = 0
        elif action < 0.4 and live:
            s = rng.choice(list(live))
            cache.free(s)
            del live[s]
        elif live:
            chosen = rng.sample(list(live), rng.randint(1, len(live)))
            amounts = [rng.choice([1, 1, 1, 7, 90]) for _ in chosen]
            try:
                cache.begin_step(chosen, amounts)
            except CacheFull:
                cache.check()
                continue
            cache.end_step(chosen, amounts)
            for s, n in zip(chosen, amounts):
                live[s] += n
        cache.check()
        for s, n in live.items():
            assert cache.length(s) == n
    for s in list(live):
        cache.free(s)
    cache.check()
    assert all(g.pool.num_held == 0 for g in cache.groups)
