"""The cache's bookkeeping on the CPU: no slot or page lost, held twice, or freed twice."""
import random

import pytest
import torch

from x0ne_engine_b200.cache import CacheFull, FreeList, SequenceCache, pages_for
from x0ne_engine_b200.parts import CacheNeed


def test_free_list_hands_out_each_item_once_and_refuses_double_free():
    f = FreeList(5, "slot")
    got = f.take(5)
    assert sorted(got) == [0, 1, 2, 3, 4] and f.available() == 0
    with pytest.raises(CacheFull):
        f.take(1)
    f.give_back([2])
    with pytest.raises(ValueError, match="twice"):
        f.give_back([2])
    with pytest.raises(ValueError):
        f.give_back([7])
    with pytest.raises(ValueError, match="twice"):
        f.give_back([0, 0])
    assert f.is_held(0) and f.take(1) == [2]


def make_cache(capacity=640, max_seq=256, slots=None, window=None):
    needs = [CacheNeed("kv", 2, 16, None), CacheNeed("kv", 2, 16, None), CacheNeed("state", state_shape=(3,))]
    if window:
        needs.append(CacheNeed("kv", 1, 8, window))
    return SequenceCache(needs, [None] * len(needs), capacity, max_seq, torch.float32, "cpu", max_slots=slots)


def test_layers_with_the_same_need_share_a_group_and_others_get_their_own():
    c = make_cache(window=40)
    assert len(c.groups) == 2
    full, win = c.groups
    assert full.entries == [0, 1] and win.entries == [3]
    assert full.storage.shape == (2, 10, 2, 2, 64, 16)
    assert win.ring_pages < full.ring_pages and c.state(2).shape == (10, 3)
    assert c.kv_view(0).base != c.kv_view(1).base and c.kv_view(0).page_table == c.kv_view(1).page_table


def test_pages_follow_the_tokens_a_sequence_holds():
    c = make_cache()
    s = c.acquire(5)
    g = c.groups[0]
    assert len(g.pages_of[s]) == 1
    c.ensure(s, 64)
    assert len(g.pages_of[s]) == 1
    c.ensure(s, 65)
    assert len(g.pages_of[s]) == 2 and g.table_host[s, :2].tolist() == g.pages_of[s]
    assert torch.equal(g.table[s, :2], torch.tensor(g.pages_of[s], dtype=torch.int32))
    with pytest.raises(CacheFull):
        c.ensure(s, 257)                      # longer than a sequence may be
    c.release(s)
    assert g.pool.available() == g.n_pages and (g.table_host[s] == -1).all()
    with pytest.raises(ValueError, match="twice"):
        c.release(s)


def test_capacity_is_counted_in_tokens_rounded_to_pages():
    c = make_cache(capacity=640)              # 10 pages
    slots = [c.acquire(64) for _ in range(10)]
    assert c.free_tokens() == 0
    with pytest.raises(CacheFull):
        c.acquire(1)
    assert c.slots.available() == 0 or c.groups[0].pool.available() == 0
    c.release(slots[3])
    assert c.acquire(33) == slots[3]          # the freed slot and page are used again


def test_a_refused_acquire_or_ensure_all_changes_nothing():
    c = make_cache(capacity=256)              # 4 pages
    a = c.acquire(128)
    before = (c.slots.available(), c.groups[0].pool.available())
    with pytest.raises(CacheFull):
        c.acquire(200)
    assert (c.slots.available(), c.groups[0].pool.available()) == before
    b = c.acquire(64)
    with pytest.raises(CacheFull):
        c.ensure_all([(a, 192), (b, 128)])    # needs 2 more pages, 1 free
    assert len(c.groups[0].pages_of[a]) == 2 and len(c.groups[0].pages_of[b]) == 1


def test_state_is_zero_when_a_slot_is_taken_again():
    c = make_cache()
    s = c.acquire(1)
    c.state(2)[s] = 5.0
    c.release(s)
    assert c.acquire(1) == s and float(c.state(2)[s].abs().sum()) == 0.0


def test_random_operations_against_a_model():
    rng = random.Random(0)
    c = make_cache(capacity=64 * 12, max_seq=64 * 5, window=70)
    held = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.4:
            want = rng.randint(0, 330)
            try:
                s = c.acquire(want)
                assert s not in held
                held[s] = want
            except CacheFull:
                pass
        elif op < 0.7 and held:
            s = rng.choice(list(held))
            want = held[s] + rng.randint(0, 100)
            try:
                c.ensure(s, want)
                held[s] = max(held[s], want)
            except CacheFull:
                pass
        elif held:
            s = rng.choice(list(held))
            c.release(s)
            del held[s]
        for g in c.groups:
            pages = [p for s in held for p in g.pages_of.get(s, [])]
            assert len(pages) == len(set(pages)), "a page is held twice"
            assert len(pages) + g.pool.available() == g.n_pages, "a page was lost"
            for s, tokens in held.items():
                assert len(g.pages_of.get(s, [])) >= g.pages_needed(tokens)
        assert c.slots.held() == len(held)
    for s in list(held):
        c.release(s)
    assert all(g.pool.available() == g.n_pages for g in c.groups) and c.slots.available() == c.n_slots


def test_pages_for():
    assert [pages_for(n) for n in (0, 1, 64, 65, 128)] == [0, 1, 1, 2, 2]
