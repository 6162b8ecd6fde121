"""The cache's bookkeeping on the CPU: no block or slot lost, held twice or
freed twice; lengths, windows, the device copy of the block table."""

import random

import pytest
import torch

from flashdecode_cuda_b200.cache import IdAllocator, KVGroupSpec, PagedCache, PoolExhausted, StateSpec


def make(num_blocks=24, slots=4, per_seq=8, bs=4, window=None, states=()):
    groups = [KVGroupSpec(2, 2, 8, None)] + ([KVGroupSpec(1, 1, 8, window)] if window else [])
    return PagedCache(groups, list(states), num_blocks, slots, per_seq, bs, torch.float32, "cpu")


def test_allocator_round_trip_lifo_exhaustion_double_free():
    a = IdAllocator(5)
    assert a.allocate(3) == [0, 1, 2] and a.num_free == 2 and a.num_used == 3
    a.free([1])
    assert a.allocate(1) == [1]                    # last freed, first reused
    with pytest.raises(PoolExhausted):
        a.allocate(3)
    assert a.num_free == 2                          # a refused request changes nothing
    a.free([0, 2])
    with pytest.raises(ValueError, match="double free"):
        a.free([0])
    with pytest.raises(ValueError, match="double free"):
        a.free([1, 1])
    assert a.in_use(1)                              # ... and the failed call freed nothing
    with pytest.raises(ValueError, match="outside"):
        a.free([7])
    assert sorted(a.allocate(a.num_free)) == [0, 2, 3, 4]


def table_on_device_matches(cache):
    cache.sync()
    for g in cache.groups:
        assert torch.equal(g.table, torch.from_numpy(g.table_host))


def test_reserve_advance_release():
    c = make()
    s = c.admit()
    assert c.length(s) == 0
    c.reserve([(s, 5)])                            # 5 tokens -> 2 blocks of 4
    assert c.blocks_in_use() == [2]
    c.reserve([(s, 5)])                            # idempotent until the length moves
    assert c.blocks_in_use() == [2]
    c.advance(s, 5)
    assert c.length(s) == 5 and c.slot_of(s, 4) == (1, 0)
    c.reserve([(s, 3)])                            # 8 tokens still fit 2 blocks
    assert c.blocks_in_use() == [2]
    c.reserve([(s, 4)])                            # 9 need a third
    assert c.blocks_in_use() == [3]
    with pytest.raises(ValueError, match="beyond"):
        c.advance(s, 9)
    table_on_device_matches(c)
    c.release(s)
    assert c.blocks_in_use() == [0] and c.active_slots() == []
    table_on_device_matches(c)
    assert int((c.groups[0].table >= 0).sum()) == 0
    with pytest.raises(ValueError, match="holds no sequence"):
        c.release(s)
    with pytest.raises(ValueError, match="holds no sequence"):
        c.length(s)
    c.check_invariants()


def test_a_slot_used_again_gets_a_clean_table_row():
    c = make()
    s = c.admit()
    c.reserve([(s, 9)])
    c.advance(s, 9)
    c.release(s)
    s2 = c.admit()
    assert s2 == s                                  # LIFO: the same slot comes back
    c.reserve([(s2, 3)])
    table_on_device_matches(c)                      # release and reuse between two syncs
    assert int((c.groups[0].table[s2] >= 0).sum()) == 1


def test_exhaustion_changes_nothing_and_limits():
    c = make(num_blocks=5)
    a, b = c.admit(), c.admit()
    c.reserve([(a, 12)])
    with pytest.raises(PoolExhausted):
        c.reserve([(a, 16), (b, 8)])                # 1 + 2 more needed, 2 free
    assert c.blocks_in_use() == [3]
    with pytest.raises(ValueError, match="table holds"):
        c.reserve([(b, 33)])                        # 9 blocks > 8 per sequence
    for _ in range(2):
        c.admit()
    with pytest.raises(PoolExhausted):
        c.admit()                                   # 4 slots
    c.check_invariants()


def test_window_group_gives_blocks_back_behind_the_window():
    c = make(num_blocks=16, per_seq=16, bs=4, window=6)
    s = c.admit()
    c.reserve([(s, 20)])
    assert c.blocks_in_use() == [5, 5]              # a whole prompt needs all its blocks during its step
    c.advance(s, 20)
    # next query at 20 sees keys 15..20: blocks 0..2 (positions 0..11) are dead
    assert c.blocks_in_use() == [5, 2]
    assert c.slot_of(s, 3, group=1)[0] == -1 and c.slot_of(s, 15, group=1)[0] >= 0
    for _ in range(12):
        c.reserve([(s, 1)])
        c.advance(s, 1)
    assert c.blocks_in_use()[1] <= 3
    table_on_device_matches(c)
    assert c.kv_bytes([s]) == 32 * c.groups[0].bytes_per_token() + 6 * c.groups[1].bytes_per_token()
    c.release(s)
    assert c.blocks_in_use() == [0, 0]
    c.check_invariants()


def test_state_is_zeroed_on_admission():
    c = make(states=[StateSpec("run0.sum", (3,), torch.float32)])
    s = c.admit()
    c.states["run0.sum"][s] += 5.0
    c.release(s)
    assert c.admit() == s
    assert float(c.states["run0.sum"][s].abs().sum()) == 0.0


def test_random_traffic_keeps_the_invariants():
    rnd = random.Random(3)
    c = make(num_blocks=40, slots=6, per_seq=10, bs=4, window=7)
    live = {}
    for step in range(600):
        op = rnd.random()
        if op < 0.25 and len(live) < 6:
            live[c.admit()] = 0
        elif op < 0.4 and live:
            s = rnd.choice(list(live))
            c.release(s)
            del live[s]
        elif live:
            s = rnd.choice(list(live))
            n = rnd.choice([1, 1, 1, 5, 9])
            if live[s] + n <= 40:
                try:
                    c.reserve([(s, n)])
                except PoolExhausted:
                    continue
                c.advance(s, n)
                live[s] += n
        if step % 50 == 0:
            c.check_invariants()
            table_on_device_matches(c)
    for s, n in live.items():
        assert c.length(s) == n
    for s in list(live):
        c.release(s)
    c.check_invariants()
    assert c.blocks_in_use() == [0, 0] and c.slot_alloc.num_used == 0


def test_lengths_version_moves_with_sequences_and_lengths_only():
    """Whoever keeps something derived from the slots' lengths (the decoder's index array filled
    ahead) compares this counter: it must move when a sequence starts, ends or grows, and must
    not move when blocks are only reserved."""
    c = make()
    v0 = c.lengths_version
    s = c.admit()
    v1 = c.lengths_version
    assert v1 != v0
    c.reserve([(s, 6)])
    c.sync()
    assert c.lengths_version == v1
    c.advance(s, 6)
    v2 = c.lengths_version
    assert v2 != v1
    c.reserve([(s, 1)])                              # the decoder's reservation for a step that may not come
    assert c.lengths_version == v2
    c.release(s)
    v3 = c.lengths_version
    assert v3 != v2
    assert c.admit() == s and c.lengths_version != v3     # the same slot with another sequence
    c.check_invariants()


def test_a_slot_listed_twice_is_refused_before_anything_changes():
    cache = PagedCache([KVGroupSpec(1, 1, 8)], [], num_blocks=8, max_slots=2, max_blocks_per_seq=4, block_size=4,
                       dtype=torch.float32, device="cpu")
    s = cache.admit()
    with pytest.raises(ValueError, match="twice"):
        cache.reserve([(s, 3), (s, 2)])
    assert cache.blocks_in_use() == [0]
    cache.check_invariants()
    cache.reserve([(s, 3)])
    cache.check_invariants()


def test_fragmentation_counts_the_unused_tails():
    cache = PagedCache([KVGroupSpec(1, 1, 8)], [], num_blocks=16, max_slots=3, max_blocks_per_seq=8, block_size=4,
                       dtype=torch.float32, device="cpu")
    assert cache.fragmentation() == 0.0
    a, b = cache.admit(), cache.admit()
    cache.reserve([(a, 5), (b, 8)])
    cache.advance(a, 5)
    cache.advance(b, 8)
    assert cache.fragmentation() == pytest.approx(1 - 13 / 16)        # a: 5 of 8 places, b: 8 of 8
    cache.release(a)
    assert cache.fragmentation() == 0.0
    assert "fragmentation" in repr(cache)
