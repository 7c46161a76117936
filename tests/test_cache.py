"""Cache bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from stratum_b200.cache import (PAGE_TOKENS, CacheFull, CacheMisuse, KVSpec, PagePool, SequenceCache,
                                SlotTable, StateSpec, pages_for)


def test_page_pool_take_give():
    pool = PagePool(4)
    a = pool.take(3)
    assert a == [0, 1, 2] and pool.free_pages == 1
    with pytest.raises(CacheFull):
        pool.take(2)
    pool.give([1])
    assert pool.take(2) == [1, 3]
    with pytest.raises(CacheMisuse):
        pool.give([1, 1])                      # second give of the same page
    pool.check()


def test_slot_table_no_double_release():
    st = SlotTable(2)
    a, b = st.acquire(), st.acquire()
    assert (a, b) == (0, 1)
    with pytest.raises(CacheFull):
        st.acquire()
    st.release(a)
    with pytest.raises(CacheMisuse):
        st.release(a)
    assert st.acquire() == 0                   # a released slot is used again
    st.check()


def _cache(max_tokens=64 * 8, max_seqs=4, specs=None):
    specs = specs if specs is not None else [KVSpec(2, 16), KVSpec(2, 16)]
    return SequenceCache(specs, max_tokens, max_seqs, torch.float32, "cpu", allocate=False)


def test_capacity_counts_rounded_up_tokens():
    c = _cache(max_tokens=64 * 4)
    s = [c.acquire() for _ in range(3)]
    c.reserve(s, [1, 64, 65])                  # 1 + 1 + 2 pages
    c.advance(s, [1, 64, 65])
    assert c.tokens_held() == 4 * PAGE_TOKENS
    with pytest.raises(CacheFull):
        c.reserve([s[1]], [1])                 # its 65th token needs a fifth page
    c.check()
    assert [c.length(x) for x in s] == [1, 64, 65]      # a refused step changes nothing
    c.release(s[2])
    c.reserve([s[1]], [1])
    c.advance([s[1]], [1])
    c.check()


def test_reserve_is_all_or_nothing():
    c = _cache(max_tokens=64 * 3)
    a, b = c.acquire(), c.acquire()
    with pytest.raises(CacheFull):
        c.reserve([a, b], [65, 65])            # 2 + 2 pages > 3
    assert c.tokens_held() == 0
    c.check()


def test_misuse_is_caught():
    c = _cache()
    a = c.acquire()
    with pytest.raises(CacheMisuse):
        c.reserve([a, a], [1, 1])
    with pytest.raises(CacheMisuse):
        c.reserve([3], [1])
    c.release(a)
    with pytest.raises(CacheMisuse):
        c.release(a)
    with pytest.raises(CacheMisuse):
        c.length(a)


def test_random_traffic_keeps_invariants():
    rng = random.Random(0)
    c = _cache(max_tokens=64 * 40, max_seqs=6)
    live = {}
    for _ in range(3000):
        r = rng.random()
        if r < 0.25 and len(live) < 6:
            live[c.acquire()] = 0
        elif r < 0.4 and live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        elif live:
            group = rng.sample(list(live), rng.randint(1, len(live)))
            n = [rng.choice([1, 1, 1, 7, 64, 130]) for _ in group]
            try:
                c.reserve(group, n)
            except CacheFull:
                continue
            c.advance(group, n)
            for s, k in zip(group, n):
                live[s] += k
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
            assert len([p for p in c.page_table_rows([s], 0)[0] if p >= 0]) == pages_for(n)
    for s in list(live):
        c.release(s)
    c.check()
    assert c.tokens_held() == 0 and c.slots.free_slots == 6


def test_groups_have_storage_of_their_own():
    specs = [KVSpec(2, 16), KVSpec(2, 16, window=100), None, StateSpec((4, 8)), KVSpec(2, 16)]
    c = SequenceCache(specs, 64 * 6, 3, torch.float32, "cpu", allocate=True)
    assert len(c.groups) == 3
    assert c.layer_group == {0: (0, 0), 1: (1, 0), 3: (2, 0), 4: (0, 1)}
    assert c.groups[0].k.shape == (2, 6, 2, PAGE_TOKENS, 16) and c.groups[1].k.shape == (1, 6, 2, PAGE_TOKENS, 16)
    assert c.groups[2].state.shape == (1, 3 + 1, 4, 8)          # a spare row for the padding rows of a step
    s = c.acquire()
    c.reserve([s], [300]); c.advance([s], [300])
    full = c.page_table_rows([s], 0)[0]
    win = c.page_table_rows([s], 1)[0]
    assert all(p >= 0 for p in full) and len(full) == 5
    # window 100: the next query (position 300) sees keys 201..300 -> pages 3 and 4 stay, 0..2 went back
    assert [p >= 0 for p in win] == [False, False, False, True, True]
    assert c.groups[1].pool.free_pages == 4
    c.check()
    # fixed-size state is zeroed when a slot is taken again
    c.groups[2].state[0, s].fill_(3.0)
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and float(c.groups[2].state[0, s2].abs().sum()) == 0.0
    v = c.layer_view(3, True, {})
    assert v.state.shape == (3 + 1, 4, 8) and v.k is None
    v = c.layer_view(2, True, {})
    assert v.spec is None
