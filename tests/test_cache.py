"""Slots, pages and stores on the host (no GPU): nothing lost, held twice or freed twice."""
import random

import pytest
import torch

from grout_b200.cache import (CacheFull, CacheLayout, KVSpec, PAGE_TOKENS, PagePool, SequenceCache,
                              SlotList, StateSpec, pages_for)


def test_free_list_invariants():
    s = SlotList(4)
    got = [s.acquire() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and len(set(got)) == 4
    with pytest.raises(CacheFull):
        s.acquire()
    s.release(2)
    with pytest.raises(ValueError):
        s.release(2)            # freed twice
    with pytest.raises(ValueError):
        s.release(9)            # never existed
    assert s.acquire() == 2     # the place given back is used again
    s.check()


def test_random_churn_keeps_every_page_accounted_for():
    rng = random.Random(0)
    p = PagePool(50)
    held = []
    for _ in range(2000):
        if held and (rng.random() < 0.5 or p.n_free == 0):
            p.release(held.pop(rng.randrange(len(held))))
        else:
            held.append(p.acquire())
        assert p.n_free + p.n_held == 50 and len(set(held)) == len(held)
    p.check()


def _cache(max_tokens=640, max_slots=4, specs=None, max_seq_len=512):
    specs = specs or [KVSpec(2, 16), KVSpec(2, 16), KVSpec(2, 16, window=100), StateSpec((3, 5))]
    layout = CacheLayout.from_specs(specs)
    return SequenceCache(layout, max_tokens=max_tokens, max_slots=max_slots, max_seq_len=max_seq_len,
                         dtype=torch.float32, device="cpu", allocate=False), layout


def test_layers_with_equal_needs_share_a_store():
    c, layout = _cache()
    assert len(layout.groups) == 3
    assert layout.where == {0: (0, 0), 1: (0, 1), 2: (1, 0), 3: (2, 0)}
    # a layer that reads another layer's cache owns nothing
    lay = CacheLayout.from_specs([KVSpec(1, 16), None, KVSpec(1, 16)])
    assert lay.where == {0: (0, 0), 2: (0, 1)} and lay.groups[0][1] == [0, 2]


def test_sequences_grow_by_pages_and_give_everything_back():
    c, _ = _cache()
    a, b = c.open(), c.open()
    c.reserve(a, 65), c.advance(a, 65)
    c.reserve(b, 1), c.advance(b, 1)
    full = c.stores[0]
    assert len(full.pages_of[a]) == 2 and len(full.pages_of[b]) == 1
    assert c.tokens_held() == 3 * PAGE_TOKENS
    for _ in range(63):
        c.reserve(a, 1), c.advance(a, 1)
    assert len(full.pages_of[a]) == 2 and c.length[a] == 128
    c.reserve(a, 1), c.advance(a, 1)
    assert len(full.pages_of[a]) == 3
    c.check()
    c.close(a)
    with pytest.raises(ValueError):
        c.close(a)              # closed twice
    with pytest.raises(ValueError):
        c.reserve(a, 1)         # not open
    c.close(b)
    c.check()
    assert c.tokens_held() == 0 and c.slots.n_held == 0


def test_window_store_frees_pages_that_fell_out_of_the_window():
    c, _ = _cache(max_seq_len=640)
    s = c.open()
    c.reserve(s, 300), c.advance(s, 300)
    win = c.stores[1]
    # window 100: keys 201.. are in reach of position 300, so pages 0..2 are gone
    assert [p is None for p in win.pages_of[s]] == [True, True, True, False, False]
    assert len([p for p in c.stores[0].pages_of[s] if p is not None]) == 5
    c.check()
    c.close(s)
    c.check()
    assert win.pool.n_held == 0


def test_limits():
    c, _ = _cache(max_tokens=128, max_slots=8)
    assert c.max_slots == 2                     # never more slots than pages
    a, b = c.open(), c.open()
    with pytest.raises(CacheFull):
        c.open()
    c.reserve(a, 64)
    c.reserve(b, 64)
    with pytest.raises(CacheFull):
        c.reserve(a, 65)                        # no page left
    c2, _ = _cache(max_seq_len=100)
    s = c2.open()
    with pytest.raises(CacheFull):
        c2.reserve(s, 101)                      # longer than the context


def test_slots_and_pages_are_reused_by_the_next_batch():
    c, _ = _cache(max_tokens=384, max_slots=4)
    first = [c.open() for _ in range(3)]
    for s in first:
        c.reserve(s, 70), c.advance(s, 70)
    pages_first = {p for s in first for p in c.stores[0].pages_of[s]}
    assert len(pages_first) == 6
    extra = c.open()
    with pytest.raises(CacheFull):
        c.reserve(extra, 70)
    c.close(extra)
    for s in first:
        c.close(s)
    second = [c.open() for _ in range(2)]
    for s in second:
        c.reserve(s, 128), c.advance(s, 128)
    assert set(second) <= set(first) | {extra}
    assert {p for s in second for p in c.stores[0].pages_of[s]} <= pages_first
    c.check()


def test_pages_for():
    assert [pages_for(n) for n in (0, 1, 64, 65, 128)] == [0, 1, 1, 2, 2]


def test_random_batches_through_the_whole_cache():
    """Sequences opened, grown by prompts and single tokens and closed in random order, with a
    full store, a window store and a state store side by side: after every operation the
    cache's own check holds, no page belongs to two sequences, and a refused request leaves
    everything as it was."""
    rng = random.Random(7)
    c, _ = _cache(max_tokens=1024, max_slots=6, max_seq_len=400)
    live = {}
    refused = 0
    for _ in range(3000):
        roll = rng.random()
        if live and roll < 0.15:
            s = rng.choice(list(live))
            c.close(s)
            del live[s]
        elif roll < 0.35:
            try:
                s = c.open()
                assert s not in live
                live[s] = 0
            except CacheFull:
                assert len(live) == c.max_slots
                refused += 1
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 17, 64, 65, 130])
            before = (c.tokens_held(), c.length[s])
            try:
                c.reserve(s, n)
                c.advance(s, n)
                live[s] += n
            except CacheFull:
                assert (c.tokens_held(), c.length[s]) == before      # nothing half done
                refused += 1
        c.check()
        for store in c.stores[:2]:
            held = [p for s in live for p in store.pages_of[s] if p is not None]
            assert len(held) == len(set(held)) == store.pool.n_held
        assert c.slots.n_held == len(live)
        for s, n in live.items():
            assert c.length[s] == n <= 400
    assert refused > 0          # the limits were met on the way
    for s in list(live):
        c.close(s)
    c.check()
    assert c.tokens_held() == 0 and c.slots.n_held == 0 and all(st.pool.n_held == 0 for st in c.stores[:2])
