import random

import pytest

from gguf_rs_cli_b200.cache import PAGE, Cache, CacheError, CacheFull, CacheLayout, FreeList, KVSpec, pages_for


def layout(window=None):
    kv = {0: KVSpec(2, 16), 1: KVSpec(2, 16), 3: KVSpec(2, 16)}
    if window:
        kv[2] = KVSpec(2, 16, window)
        kv[4] = KVSpec(2, 16, window)
    return CacheLayout(kv=kv, states={"s": ((4,), "float32")})


def test_free_list_refuses_misuse():
    f = FreeList(3, "slot")
    a = f.take(2)
    assert a == [0, 1] and f.free_count == 1
    with pytest.raises(CacheFull):
        f.take(2)
    assert f.free_count == 1                      # nothing was taken
    f.give_back([0])
    with pytest.raises(CacheError, match="twice"):
        f.give_back([0])
    with pytest.raises(CacheError, match="does not exist"):
        f.give_back([7])
    with pytest.raises(CacheError, match="twice"):
        f.give_back([1, 1])
    assert f.take(1) == [0]                        # lowest first: reuse shows early
    f.check()


def test_groups_by_need():
    c = Cache(layout(window=100), n_slots=4, n_tokens=64 * 40, max_len=64 * 20, max_step_tokens=64)
    assert len(c.groups) == 2
    full, win = c.groups
    assert full.runs == [0, 1, 3] and win.runs == [2, 4]
    assert full.ring_pages == 20 and full.n_pages == 40
    assert win.ring_pages == pages_for(100 + 63) + 1 == 4 and win.n_pages == 16
    assert c.group_of_run[3] == (0, 2) and c.group_of_run[4] == (1, 1)


def test_reserve_is_all_or_nothing_and_lengths_are_per_sequence():
    c = Cache(layout(), n_slots=3, n_tokens=64 * 6)
    a, b = c.open(), c.open()
    c.reserve([a, b], [65, 1])
    c.advance([a, b], [65, 1])
    assert c.length(a) == 65 and c.length(b) == 1
    assert len(c.groups[0].tables[a]) == 2 and len(c.groups[0].tables[b]) == 1
    with pytest.raises(CacheFull):
        c.reserve([a, b], [64, 64 * 3])            # b alone would need 3 more, a one more: 4 > 3 free
    assert c.groups[0].pool.free_count == 3 and len(c.groups[0].tables[a]) == 2
    c.reserve([a], [63])                           # 128 positions still fit two pages
    assert len(c.groups[0].tables[a]) == 2
    with pytest.raises(CacheError, match="twice"):
        c.reserve([a, a], [1, 1])
    with pytest.raises(CacheError, match="not open"):
        c.reserve([2], [1])
    c.check()


def test_close_gives_everything_back_and_slots_are_reused():
    c = Cache(layout(window=70), n_slots=2, n_tokens=64 * 8, max_step_tokens=64)
    a = c.open()
    c.reserve([a], [64]); c.advance([a], [64])
    c.reserve([a], [64]); c.advance([a], [64])
    held = [g.pool.held_count for g in c.groups]
    assert held[0] == 2
    c.close(a)
    assert [g.pool.held_count for g in c.groups] == [0, 0] and c.slots.held_count == 0
    with pytest.raises(CacheError, match="not open"):
        c.close(a)
    assert c.open() == a and c.length(a) == 0
    c.check()


def test_window_group_keeps_a_ring():
    c = Cache(layout(window=70), n_slots=2, n_tokens=64 * 32, max_step_tokens=64)
    win = c.groups[1]
    ring = win.ring_pages
    a = c.open()
    for _ in range(20):
        c.reserve([a], [64]); c.advance([a], [64])
    assert len(win.tables[a]) == ring and len(c.groups[0].tables[a]) == 20
    with pytest.raises(CacheFull, match="one step"):
        c.reserve([a], [65])
    c.check()


def test_random_walk_loses_nothing():
    rng = random.Random(0)
    c = Cache(layout(window=90), n_slots=5, n_tokens=64 * 24, max_len=64 * 10, max_step_tokens=128)
    live = []
    for _ in range(600):
        r = rng.random()
        try:
            if r < 0.25 and c.slots.free_count:
                live.append(c.open())
            elif r < 0.45 and live:
                c.close(live.pop(rng.randrange(len(live))))
            elif live:
                k = rng.randint(1, len(live))
                slots = rng.sample(live, k)
                n = [rng.randint(1, 128) for _ in slots]
                c.reserve(slots, n)
                c.advance(slots, n)
        except CacheFull:
            pass
        c.check()
        assert c.tokens_held() <= 64 * 24
    for s in live:
        c.close(s)
    c.check()
    assert all(g.pool.held_count == 0 for g in c.groups) and c.slots.held_count == 0
