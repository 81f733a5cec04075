"""The cache's bookkeeping (no GPU): no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from burn_transformers_b200.cache import CacheBank, CacheConfig, CacheNeed, FreeList, KvSpec, StateSpec, PAGE_SIZE
from burn_transformers_b200.errors import CacheError


def bank(max_tokens=512, max_slots=4, max_context=256, needs=None):
    needs = needs or [CacheNeed(kv=KvSpec(2, 16)), CacheNeed(kv=KvSpec(2, 16)),
                      CacheNeed(kv=KvSpec(1, 32, window=70), states=(StateSpec("sum", (3,)),))]
    return CacheBank(needs, CacheConfig(max_tokens, max_slots, max_context), torch.float32, "cpu")


def test_free_list():
    pool = FreeList(3, "slot")
    a, b, c = pool.take(), pool.take(), pool.take()
    assert sorted((a, b, c)) == [0, 1, 2] and pool.free == 0
    with pytest.raises(CacheError, match="no free slot"):
        pool.take()
    pool.give_back(b)
    with pytest.raises(CacheError, match="freed twice"):
        pool.give_back(b)
    with pytest.raises(CacheError, match="does not exist"):
        pool.give_back(7)
    assert pool.take() == b
    pool.check()


def test_groups_have_storage_of_their_own():
    b = bank()
    assert len(b.groups) == 2
    full, ring = b.groups
    assert full.k.shape == (2, 8, 2, PAGE_SIZE, 16) and not full.is_ring and full.table_len == 4
    assert ring.k.shape[0] == 1 and ring.is_ring and ring.table_len == 2      # window 70 spans two pages
    assert ring.k.shape[1] == min(8, 4 * 2)
    assert b.entry_group(1) == (0, 1) and b.entry_group(2) == (1, 0)
    assert b.state(2, "sum").shape == (4, 3)


def test_reserve_commit_release():
    b = bank()
    s = b.acquire()
    b.reserve([(s, 65)])
    assert len(b.table_row(0, s)) == 2 and len(b.table_row(1, s)) == 2
    assert b.length(s) == 0                      # lengths move only on commit
    b.commit(s, 65)
    b.reserve([(s, 200)])
    assert len(b.table_row(0, s)) == 4 and len(b.table_row(1, s)) == 2   # the ring never grows past its window
    b.commit(s, 200)
    assert b.tokens_held() == 256
    with pytest.raises(CacheError, match="exceed the longest sequence"):
        b.reserve([(s, 257)])
    with pytest.raises(CacheError, match="cannot shrink"):
        b.reserve([(s, 10)])
    b.state(2, "sum")[s] = 5.0
    b.release(s)
    assert float(b.state(2, "sum")[s].abs().sum()) == 0.0       # state is zeroed when a slot is given back
    with pytest.raises(CacheError, match="released twice"):
        b.release(s)
    with pytest.raises(CacheError, match="not in use"):
        b.length(s)
    b.check()
    assert b.groups[0].pool.free == 8 and b.groups[1].pool.free == 8


def test_full_cache_changes_nothing():
    b = bank(max_tokens=256)
    s1, s2 = b.acquire(), b.acquire()
    b.reserve([(s1, 128)])
    b.commit(s1, 128)
    before = [list(b.table_row(0, s)) for s in (s1, s2)]
    with pytest.raises(CacheError, match="cache is full"):
        b.reserve([(s1, 129), (s2, 100)])        # 1 + 2 pages wanted, 2 free
    assert [list(b.table_row(0, s)) for s in (s1, s2)] == before
    b.check()


def test_random_traffic_keeps_the_books():
    rng = random.Random(3)
    b = bank(max_tokens=64 * 12, max_slots=5, max_context=64 * 6)
    live = {}
    for _ in range(600):
        action = rng.random()
        if action < 0.3 and len(live) < 5:
            live[b.acquire()] = 0
        elif action < 0.8 and live:
            s = rng.choice(list(live))
            want = min(64 * 6, live[s] + rng.choice([1, 1, 1, 17, 64, 130]))
            try:
                b.reserve([(s, want)])
                b.commit(s, want)
                live[s] = want
            except CacheError:
                pass
        elif live:
            s = rng.choice(list(live))
            b.release(s)
            del live[s]
        b.check()
        for s, n in live.items():
            assert b.length(s) == n
            assert len(b.table_row(0, s)) >= -(-n // PAGE_SIZE)
        pages = [p for s in live for p in b.table_row(0, s)]
        assert len(pages) == len(set(pages))
    for s in list(live):
        b.release(s)
    b.check()
    assert b.slots.free == 5 and all(g.pool.held == 0 for g in b.groups)


def test_config_rejects_zero():
    with pytest.raises(CacheError):
        CacheConfig(0, 1, 1)
