"""Slot and page bookkeeping of the cache (no GPU, no storage)."""
import random

import pytest
import torch

from wick_b200.cache import PAGE, Cache, CacheFull, IndexPool, PoolError, PoolExhausted
from wick_b200.parts.base import CacheNeed

KV = CacheNeed("paged_kv", kv_heads=2, head_dim=16)


def make(max_tokens=640, layers=3, **kw):
    return Cache([KV] * layers, max_tokens=max_tokens, dtype=torch.float32, device="cpu", allocate=False, **kw)


def test_index_pool_hands_out_lowest_first_and_never_twice():
    p = IndexPool(5, reserved=(0,))
    assert [p.alloc() for _ in range(4)] == [1, 2, 3, 4]
    with pytest.raises(PoolExhausted):
        p.alloc()
    p.free(3)
    p.free(1)
    assert p.alloc() == 1 and p.alloc() == 3
    p.check()


def test_index_pool_refuses_double_free_and_foreign_indices():
    p = IndexPool(4, reserved=(0,))
    a = p.alloc()
    p.free(a)
    with pytest.raises(PoolError, match="freed twice"):
        p.free(a)
    with pytest.raises(PoolError, match="does not belong"):
        p.free(0)
    with pytest.raises(PoolError, match="does not belong"):
        p.free(17)
    p.check()


def test_pages_follow_length_in_units_of_64():
    c = make(max_tokens=640)
    assert c.n_pages == 11 and c.pages.capacity == 10 and c.free_tokens == 640
    s = c.open_seq()
    assert s != 0, "slot 0 is kept for padding"
    c.reserve(s, 1)
    assert len(c.pages_of(s)) == 1 and 0 not in c.pages_of(s)
    c.reserve(s, 64)
    assert len(c.pages_of(s)) == 1
    c.reserve(s, 65)
    assert len(c.pages_of(s)) == 2
    c.advance(s, 65)
    assert c.length(s) == 65
    with pytest.raises(PoolError, match="holds 2 pages"):
        c.advance(s, 64)
    c.check()
    c.close_seq(s)
    assert c.pages.n_free == 10 and c.slots.n_held == 0
    c.check()


def test_full_cache_and_context_limit():
    c = make(max_tokens=128, max_position=100)
    a, b = c.open_seq(), c.open_seq()
    c.reserve(a, 64)
    c.reserve(b, 64)
    with pytest.raises(CacheFull, match="the cache is full"):
        c.reserve(b, 65)
    with pytest.raises(PoolExhausted, match="no free slot"):
        c.open_seq()                      # at most one sequence per page
    with pytest.raises(ValueError, match="context length exceeded"):
        c.reserve(a, 101)
    c.close_seq(a)
    c.reserve(b, 65)
    c.check()


def test_closing_twice_and_using_a_closed_slot_fail():
    c = make()
    s = c.open_seq()
    c.close_seq(s)
    with pytest.raises(PoolError, match="closed twice"):
        c.close_seq(s)
    with pytest.raises(PoolError, match="not open"):
        c.length(s)
    with pytest.raises(PoolError, match="not open"):
        c.reserve(s, 3)


def test_slots_and_pages_are_used_again():
    c = make(max_tokens=256)
    s1 = c.open_seq()
    c.reserve(s1, 200)
    first = list(c.pages_of(s1))
    c.close_seq(s1)
    s2 = c.open_seq()
    c.reserve(s2, 100)
    assert s2 == s1 and c.pages_of(s2) == first[:2], "freed slots and pages come back first"
    assert c.length(s2) == 0, "a reused slot starts empty"


def test_truncate_gives_pages_back():
    c = make(max_tokens=512)
    s = c.open_seq()
    c.reserve(s, 300)
    c.advance(s, 300)
    c.truncate(s, 70)
    assert c.length(s) == 70 and len(c.pages_of(s)) == 2
    c.check()
    with pytest.raises(ValueError):
        c.truncate(s, 71)


def test_random_traffic_loses_nothing_and_shares_nothing():
    rng = random.Random(0)
    c = make(max_tokens=64 * 40, max_seqs=12)
    live = {}
    for step in range(3000):
        r = rng.random()
        if r < 0.25 and c.slots.n_free:
            s = c.open_seq()
            assert s not in live
            live[s] = 0
        elif r < 0.75 and live:
            s = rng.choice(list(live))
            n = rng.randint(1, 150)
            try:
                c.reserve(s, live[s] + n)
            except CacheFull:
                continue
            c.advance(s, n)
            live[s] += n
            assert c.length(s) == live[s]
        elif live:
            s = rng.choice(list(live))
            c.close_seq(s)
            del live[s]
        if step % 50 == 0:
            c.check()
            pages = [p for s in live for p in c.pages_of(s)]
            assert len(pages) == len(set(pages)) and 0 not in pages
            assert c.pages.n_held == len(pages)
            assert all(len(c.pages_of(s)) == -(-live[s] // PAGE) for s in live)
    for s in list(live):
        c.close_seq(s)
    c.check()
    assert c.pages.n_held == 0 and c.slots.n_held == 0


def test_groups_by_need_and_fixed_size_state():
    needs = [KV, CacheNeed("state", shape=(4, 8), dtype=torch.float32), KV, None,
             CacheNeed("paged_kv", kv_heads=1, head_dim=32), CacheNeed("state", shape=(4, 8), dtype=torch.float32)]
    c = Cache(needs, max_tokens=128, dtype=torch.float32, device="cpu", max_seqs=3)
    assert len(c.groups) == 3
    kv0, st, kv1 = c.groups
    assert kv0.entries == [0, 2] and st.entries == [1, 5] and kv1.entries == [4]
    assert kv0.storage.shape == (2, 3, 2, 2, PAGE, 16) and kv1.storage.shape == (1, 3, 2, 1, PAGE, 32)
    assert st.storage.shape == (2, 4, 4, 8)
    assert c.view(3) is None and c.view(0).kv.shape == (3, 2, 2, PAGE, 16)
    assert c.view(2).kv.data_ptr() != c.view(0).kv.data_ptr()
    s = c.open_seq()
    c.view(5).state[s].fill_(3.0)
    c.close_seq(s)
    s2 = c.open_seq()
    assert s2 == s and float(c.view(5).state[s2].abs().sum()) == 0.0, "state is zeroed when a sequence opens"
    assert c.bytes_per_token() == (2 * 2 * 2 * 16 + 1 * 2 * 1 * 32) * 4


def test_windowed_storage_is_refused_clearly():
    with pytest.raises(ValueError, match="a window needs a storage kind of its own"):
        Cache([CacheNeed("paged_kv", kv_heads=1, head_dim=16, window=128)], max_tokens=64, dtype=torch.float32,
              device="cpu", allocate=False)
    with pytest.raises(ValueError, match="unknown cache need ring"):
        Cache([CacheNeed("ring", kv_heads=1, head_dim=16, window=128)], max_tokens=64, dtype=torch.float32,
              device="cpu", allocate=False)


def test_a_storage_kind_registered_from_outside_gets_its_group():
    """Another kind of storage is an addition: a class registered under a new kind name
    serves every need of that kind, beside the groups of the kinds that are built in."""
    from wick_b200.cache import CacheView, Storage, register_storage

    class LastPositions(Storage):
        kind = "test_ring"

        def shape(self):
            n = self.need
            return (self.n_entries, self.n_slots, 2, n.kv_heads, n.window, n.head_dim)

        def view(self, idx, batch):
            return CacheView(ring=self.tensor[idx], window=self.need.window)

        def read_bytes(self, cached_tokens, n_seqs):
            n = self.need
            return n_seqs * self.n_entries * 2 * n.kv_heads * n.window * n.head_dim * self.element_size()

    register_storage("test_ring", LastPositions)
    needs = [CacheNeed("paged_kv", kv_heads=2, head_dim=16), CacheNeed("test_ring", kv_heads=1, head_dim=8, window=4),
             CacheNeed("test_ring", kv_heads=1, head_dim=8, window=4), CacheNeed("state", shape=(5,), dtype=torch.float32)]
    c = Cache(needs, max_tokens=128, dtype=torch.float32, device="cpu", max_seqs=3)
    assert [g.need.kind for g in c.groups] == ["paged_kv", "test_ring", "state"]
    assert c.groups[1].storage.shape == (2, 4, 2, 1, 4, 8)
    v = c.view(2)
    assert v.window == 4 and v.ring.shape == (4, 2, 1, 4, 8) and v.kv is None
    # a decode step of 3 sequences holding 100 positions: the paged group reads by position,
    # the ring by its window, the records by sequence
    assert c.read_bytes(100, 3) == 100 * 2 * 2 * 16 * 4 + 3 * 2 * 2 * 1 * 4 * 8 * 4 + 3 * 5 * 4
    assert c.bytes_per_token() == 2 * 2 * 16 * 4
