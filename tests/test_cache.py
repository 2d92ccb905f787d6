"""The cache's bookkeeping: slots, pages, lengths, groups, state."""
import random

import numpy as np
import pytest
import torch

from math_utils_b200.cache import CacheError, CacheFull, SequenceCache, SlotAllocator
from math_utils_b200.parts import KVCacheSpec, StateCacheSpec


def test_slots_are_never_lost_or_held_twice():
    a = SlotAllocator(5)
    rng = random.Random(0)
    held = []
    for _ in range(2000):
        if held and (rng.random() < 0.5 or a.n_free == 0):
            a.release(held.pop(rng.randrange(len(held))))
        else:
            s = a.acquire()
            assert s not in held
            held.append(s)
        assert len(held) + a.n_free == 5 and a.held == frozenset(held)
    with pytest.raises(CacheError, match="not held"):
        a.release(next(s for s in range(5) if s not in held) if len(held) < 5 else 99)
    while a.n_free:
        held.append(a.acquire())
    with pytest.raises(CacheFull):
        a.acquire()
    a.release(held[0])
    with pytest.raises(CacheError, match="freed twice"):
        a.release(held[0])


def make_cache(max_tokens=512, max_positions=200, specs=None, n_slots=None):
    specs = specs if specs is not None else [KVCacheSpec(2, 16), KVCacheSpec(2, 16)]
    return SequenceCache(specs, max_tokens, max_positions, torch.float32, "cpu", n_slots=n_slots)


def test_pages_follow_lengths_and_come_back():
    c = make_cache(max_tokens=512)                    # 8 pages of 64
    assert c.n_pages == 8 and c.n_slots == 8 and len(c.kv_groups) == 1
    s = c.acquire()
    assert c.reserve(s, 65) == 0
    c.commit(s, 65)
    assert c.length(s) == 65 and c.kv_groups[0].pages_held(s) == 2 and c.free_pages() == 6
    for _ in range(63):
        c.reserve(s, 1); c.commit(s, 1)
    assert c.length(s) == 128 and c.kv_groups[0].pages_held(s) == 2
    c.reserve(s, 1); c.commit(s, 1)
    assert c.kv_groups[0].pages_held(s) == 3
    t = c.acquire()
    c.reserve(t, 200); c.commit(t, 200)
    assert c.free_pages() == 8 - 3 - 4
    rows = c.block_table_rows(0, [t, s])
    assert rows.shape == (2, 4) and len(set(rows[0].tolist()) | set(rows[1][:3].tolist())) == 7
    with pytest.raises(CacheError, match="exceed"):
        c.reserve(t, 1)
    u = c.acquire()
    with pytest.raises(CacheFull):
        c.reserve(u, 65)                              # one page is left, two are needed
    c.release(s)
    c.reserve(u, 65); c.commit(u, 65)
    c.release(t); c.release(u)
    assert c.free_pages() == 8 and c.slots.n_free == 8
    with pytest.raises(CacheError):
        c.release(u)
    with pytest.raises(CacheError):
        c.length(u)


def test_groups_by_need_and_window_gives_pages_back():
    full, win = KVCacheSpec(2, 16, 0), KVCacheSpec(2, 16, 70)
    c = make_cache(max_tokens=1024, max_positions=600, specs=[full, win, None, full, StateCacheSpec(6)])
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    assert c.kv_groups[0].entries == [0, 3] and c.kv_groups[1].entries == [1]
    assert c.entry(2) is None and c.entry(0).group == 0 and c.entry(1).group == 1
    assert c.entry(0).pages.shape == (16, 2, 2, 64, 16)
    s = c.acquire()
    c.reserve(s, 300); c.commit(s, 300)
    assert c.kv_groups[0].pages_held(s) == 5
    # the next query (position 300) sees keys 231..300: page index 3 and on
    assert c.kv_groups[1].pages_held(s) == 2
    for _ in range(100):
        c.reserve(s, 1); c.commit(s, 1)
    assert c.kv_groups[0].pages_held(s) == 7 and c.kv_groups[1].pages_held(s) <= 3
    c.release(s)
    assert c.free_pages(0) == 16 and c.free_pages(1) == 16


def test_state_is_zero_for_a_new_sequence():
    c = make_cache(specs=[StateCacheSpec(4)], n_slots=2)
    s = c.acquire()
    view = c.entry(0)
    view.values[s] += 3.0
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and float(view.values[s2].abs().sum()) == 0.0


def test_random_traffic_conserves_pages():
    c = make_cache(max_tokens=64 * 40, max_positions=500, n_slots=10)
    rng = random.Random(1)
    live = {}
    for _ in range(3000):
        if live and rng.random() < 0.15:
            s = rng.choice(list(live)); c.release(s); del live[s]
        elif len(live) < 10 and rng.random() < 0.3:
            live[c.acquire()] = 0
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 17, 64])
            if live[s] + n <= 500:
                try:
                    c.reserve(s, n); c.commit(s, n); live[s] += n
                except CacheFull:
                    pass
        held = sum(c.kv_groups[0].pages_held(s) for s in live)
        assert held + c.free_pages() == c.n_pages
        for s, n in live.items():
            assert c.length(s) == n and c.kv_groups[0].pages_held(s) >= -(-n // 64)
        tables = [set(c.kv_groups[0].table[s][c.kv_groups[0].table[s] >= 0].tolist()) for s in live]
        assert sum(len(t) for t in tables) == len(set().union(*tables)) if tables else True
