"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""

import random

import pytest
import torch

from starter_b200.cache import CacheFull, IndexAllocator, KVNeed, SequenceCache, StateNeed, pages_for


def test_allocator_hands_out_each_number_once_and_refuses_double_free():
    a = IndexAllocator(5, "slot")
    got = [a.take() for _ in range(5)]
    assert sorted(got) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheFull):
        a.take()
    a.give_back(3)
    with pytest.raises(ValueError):
        a.give_back(3)
    with pytest.raises(ValueError):
        a.give_back(7)
    assert a.take() == 3
    a.check()
    with pytest.raises(CacheFull):
        a.take_many(1)
    assert a.held_count == 5 and a.free_count == 0


def make_cache(max_tokens=64 * 10, seqs=4):
    kv = {0: KVNeed(2, 16), 1: KVNeed(2, 16), 2: KVNeed(2, 16, window=8), 3: KVNeed(1, 32)}
    state = {0: None, 1: StateNeed((3, 5)), 2: None, 3: None}
    return SequenceCache(kv, state, max_tokens, seqs, torch.float32, "cpu")


def test_groups_have_storage_of_their_own():
    c = make_cache()
    assert [(g.need, g.entries) for g in c.groups] == [
        (KVNeed(2, 16), [0, 1]), (KVNeed(2, 16, 8), [2]), (KVNeed(1, 32), [3])]
    assert c.keys[0].shape == (2, 10, 2, 64, 16) and c.keys[2].shape == (1, 10, 1, 64, 32)
    k0, _ = c.entry_pages(0)
    k1, _ = c.entry_pages(1)
    assert k0.data_ptr() != k1.data_ptr() and k0.shape == (10, 2, 64, 16)
    assert c.entry_state(1).shape == (4, 3, 5) and c.entry_state(0) is None
    assert c.bytes_per_token() == 2 * 4 * (2 * 2 * 16 + 2 * 16 + 32)


def test_sequences_take_pages_as_they_grow_and_give_everything_back():
    c = make_cache()
    s = c.open_sequence()
    c.reserve(s, 65)
    assert len(c.owned_pages(s)) == 2 and c.pages.free_count == 8
    assert c.advance(s, 65) == 0 and c.lengths[s] == 65
    with pytest.raises(CacheFull):
        c.advance(s, 64)                       # would need a third page: reserve first
    c.reserve(s, 129)
    c.sync_table()
    assert c.block_table[s, :3].tolist() == c.owned_pages(s)
    c.check()
    c.close_sequence(s)
    with pytest.raises(ValueError):
        c.close_sequence(s)
    assert c.pages.free_count == 10 and c.slots.free_count == 4
    c.check()


def test_state_is_zero_when_a_slot_is_used_again():
    c = make_cache()
    s = c.open_sequence()
    c.entry_state(1)[s] += 7
    c.close_sequence(s)
    t = c.open_sequence()
    assert t == s and c.entry_state(1)[t].abs().sum() == 0 and c.lengths[t] == 0


def test_exhaustion_changes_nothing():
    c = make_cache(max_tokens=64 * 3, seqs=2)
    a, b = c.open_sequence(), c.open_sequence()
    with pytest.raises(CacheFull):
        c.open_sequence()
    c.reserve(a, 128)
    with pytest.raises(CacheFull):
        c.reserve(b, 129)
    assert c.owned_pages(b) == [] and c.pages.free_count == 1
    c.check()


def test_random_open_grow_close_never_loses_or_doubles_anything():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 40, seqs=6)
    live = {}
    for _ in range(2000):
        move = rng.random()
        try:
            if move < 0.3 and len(live) < 6:
                live[c.open_sequence()] = 0
            elif move < 0.8 and live:
                s = rng.choice(list(live))
                n = rng.randint(1, 150)
                c.reserve(s, live[s] + n)
                c.advance(s, n)
                live[s] += n
            elif live:
                s = rng.choice(list(live))
                c.close_sequence(s)
                del live[s]
        except CacheFull:
            pass
        c.check()
        assert c.pages.held_count == sum(len(c.owned_pages(s)) for s in live)
        for s, n in live.items():
            assert c.lengths[s] == n and len(c.owned_pages(s)) >= pages_for(n)
    pages = [p for s in live for p in c.owned_pages(s)]
    assert len(pages) == len(set(pages)) == c.pages.held_count
