"""The cache's bookkeeping: no slot or page is lost, held twice or freed twice; groups
with a window have storage of their own; states are zeroed when a slot is handed out."""
from __future__ import annotations

import random

import pytest
import torch

from toyinfer_b200.cache import CacheError, CacheManager, PAGE, PagePool, SlotAllocator, pages_for
from toyinfer_b200.parts.base import KVRequest, StateRequest


def test_slot_allocator_never_hands_out_twice():
    a = SlotAllocator(5)
    got = [a.allocate() for _ in range(5)]
    assert sorted(got) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheError):
        a.allocate()
    a.release(3)
    with pytest.raises(CacheError):
        a.release(3)
    with pytest.raises(CacheError):
        a.release(9)
    assert a.allocate() == 3


def test_page_pool_accounting():
    p = PagePool(6)
    x = p.allocate(4)
    assert 0 not in x and len(set(x)) == 4
    with pytest.raises(CacheError):
        p.allocate(3)
    p.release(x[:2])
    with pytest.raises(CacheError):
        p.release(x[:1])
    assert p.n_free == 4


def make(window=0, max_tokens=64 * 10, n_slots=4, max_seq_len=400):
    reqs = [KVRequest(2, 16, 0), None, KVRequest(2, 16, window), StateRequest((3, 2)), KVRequest(2, 16, 0)]
    return CacheManager(reqs, max_tokens, n_slots, max_seq_len, torch.float32, "cpu")


def test_groups_have_storage_of_their_own():
    c = make(window=100)
    assert len(c.kv_groups) == 2
    full = next(g for g in c.kv_groups if not g.ring_pages)
    ring = next(g for g in c.kv_groups if g.ring_pages)
    assert full.entries == [0, 4] and ring.entries == [2]
    assert ring.ring_rows == 128 and ring.pages_per_seq == 2
    assert full.k.shape == (2, 11, 2, PAGE, 16) and ring.k.shape == (1, 9, 2, PAGE, 16)   # min(10, 4 slots * 2) + scratch
    assert c.view(1) is None and c.view(3).state.shape == (5, 3, 2)
    assert c.view(0).k_pages.data_ptr() != c.view(4).k_pages.data_ptr()
    assert c.view(0).page_table.data_ptr() == c.view(4).page_table.data_ptr()
    assert c.view(2).ring_rows == 128 and c.view(0).ring_rows == 0


def test_pages_follow_lengths_and_come_back():
    c = make(window=100)
    full = next(g for g in c.kv_groups if not g.ring_pages)
    ring = next(g for g in c.kv_groups if g.ring_pages)
    s = c.allocate_slot()
    c.reserve(s, 1)
    assert len(full.slot_pages[s]) == 1 and len(ring.slot_pages[s]) == 1
    c.reserve(s, 65)
    c.reserve(s, 300)
    assert len(full.slot_pages[s]) == 5 and len(ring.slot_pages[s]) == 2
    c.flush()
    assert c.view(0).page_table[s, :5].tolist() == full.slot_pages[s]
    assert (c.view(0).page_table[s, 5:] == 0).all()
    with pytest.raises(CacheError):
        c.reserve(s, 401)                      # beyond max_seq_len
    t = c.allocate_slot()
    with pytest.raises(CacheError):
        c.reserve(t, 64 * 6)                   # 5 + 6 pages > 10
    c.release(s)
    with pytest.raises(CacheError):
        c.release(s)
    with pytest.raises(CacheError):
        c.reserve(s, 5)
    c.reserve(t, 64 * 6)
    c.release(t)
    assert full.pool.n_free == full.pool.n_pages and ring.pool.n_free == ring.pool.n_pages
    assert c.slots.n_free == 4 and not c.length


def test_state_is_zero_for_a_new_sequence():
    c = make()
    s = c.allocate_slot()
    c.view(3).state[s] += 5
    c.release(s)
    s2 = c.allocate_slot()
    assert s2 == s and (c.view(3).state[s2] == 0).all()


def test_random_traffic_keeps_the_books():
    rnd = random.Random(0)
    c = make(window=70, max_tokens=64 * 40, n_slots=6)
    live = {}
    for _ in range(2000):
        op = rnd.random()
        if op < 0.3 and len(live) < 6:
            live[c.allocate_slot()] = 0
        elif op < 0.8 and live:
            s = rnd.choice(list(live))
            n = min(400, live[s] + rnd.choice([1, 1, 1, 30, 90]))
            try:
                c.reserve(s, n)
                c.commit(s, n)
                live[s] = n
            except CacheError:
                pass
        elif live:
            s = rnd.choice(list(live))
            c.release(s)
            del live[s]
        for g in c.kv_groups:
            held = [p for pages in g.slot_pages.values() for p in pages]
            assert len(held) == len(set(held)) and 0 not in held
            assert len(held) + g.pool.n_free == g.pool.n_pages
            for s, n in live.items():
                assert len(g.slot_pages.get(s, [])) >= g.pages_needed(n)
        assert set(live) == set(c.length) and c.slots.n_free == 6 - len(live)
        assert c.tokens_held() == sum(pages_for(n) * PAGE for n in live.values())
