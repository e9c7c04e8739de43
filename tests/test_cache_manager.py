"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; groups with a window give pages back early; state slots."""
import random

import pytest
import torch

from tiny_transformer_inference_engine_b200.cache import PageAllocator, OutOfPages, CacheManager, pages_for
from tiny_transformer_inference_engine_b200.parts.base import PagedKVNeed, FixedStateNeed, RunEntry


def test_allocator_contract():
    # serving/allocator.py and tests/test_block_allocator.py:4-33 of the reference
    a = PageAllocator(5)
    assert a.num_usable == 4 and a.num_free == 4
    got = a.allocate_n(4)
    assert sorted(got) == [1, 2, 3, 4] and got[0] == 1           # ascending on first use, page 0 never
    with pytest.raises(OutOfPages):
        a.allocate()
    a.free([2])
    assert a.allocate() == 2                                      # a freed page is the next one used
    with pytest.raises(ValueError):
        a.free([0])
    with pytest.raises(ValueError):
        a.free([9])
    a.free([3])
    with pytest.raises(ValueError):
        a.free([3])
    before = a.num_free
    with pytest.raises(ValueError):
        a.free([1, 4, 1])                                         # a failed free changes nothing
    assert a.num_free == before
    with pytest.raises(OutOfPages):
        a.allocate_n(3)
    assert a.num_free == before


def manager(needs, order=None, page=4, pages=9, slots=3):
    order = order or [RunEntry(i) for i in range(len(needs))]
    return CacheManager(needs, order, page, pages, slots, "float32", "cpu", allocate=True)


def test_tables_slots_and_release():
    need = PagedKVNeed(1, 8)
    m = manager([need, need])
    assert len(m.groups) == 1 and m.groups[0].kv.shape == (2, 2, 9, 1, 4, 8)
    s = m.admit("a")
    m.extend("a", 0, 5)
    assert m.table(0, "a") == [1, 2] and m.num_free_pages == 6
    m.extend("a", 5, 8)                                           # still inside page 2
    assert m.table(0, "a") == [1, 2]
    m.extend("a", 8, 9)                                           # grows at the page edge
    assert m.table(0, "a") == [1, 2, 3]
    m.admit("b"); m.extend("b", 0, 4)
    assert set(m.table(0, "a")).isdisjoint(m.table(0, "b"))
    with pytest.raises(ValueError):
        m.admit("a")
    m.admit("c")
    assert not m.can_admit()
    with pytest.raises(OutOfPages):
        m.admit("d")
    m.check()
    with pytest.raises(OutOfPages):
        m.extend("c", 0, 4 * 5)                                   # 5 pages wanted, 4 free
    assert m.num_free_pages == 4 and m.table(0, "c") == []        # nothing taken by the failed call
    m.release("a")
    assert m.num_free_pages == 7 and m.slots.num_free == 1
    with pytest.raises(KeyError):
        m.release("a")
    m.admit("d")
    assert m.slot_of["d"] == s                                    # the slot is used again
    m.extend("d", 0, 3)
    assert m.table(0, "d") == [3]                                 # and so is the page freed last (LIFO)
    m.check()


def test_groups_and_window():
    full, win = PagedKVNeed(1, 8), PagedKVNeed(1, 8, window=6)
    m = manager([full, win, full, None], page=4, pages=6)
    assert len(m.groups) == 2 and m.groups[0].entries == [0, 2] and m.groups[1].entries == [1]
    m.admit("a")
    m.extend("a", 0, 10)
    assert m.table(0, "a") == [1, 2, 3] and m.table(1, "a") == [1, 2, 3]
    # next token at position 10 reads keys 5..10 in the windowed group: page 0 (keys 0..3) can go
    m.extend("a", 10, 11)
    assert m.table(1, "a") == [0, 2, 3] and m.table(0, "a") == [1, 2, 3]
    assert m.groups[1].allocator.num_free == 3 and m.groups[0].allocator.num_free == 2
    m.extend("a", 11, 16)                                         # keys from 11-6+1=6 on: page 1 holds 4..7, stays
    assert m.table(1, "a") == [0, 2, 3, 1]                        # the page given back is used again
    m.extend("a", 16, 17)                                         # keys 11..16: pages 0,1 gone
    assert m.table(1, "a") == [0, 0, 3, 1, 2]
    m.check()
    m.release("a")
    assert all(g.allocator.num_free == g.allocator.num_usable for g in m.groups)


def test_state_slots_are_zeroed():
    m = manager([PagedKVNeed(1, 8), FixedStateNeed((3,))], slots=2)
    state = m.entry_state[1]
    assert state.shape == (2, 3)
    a = m.admit("a")
    state[a] += 5
    m.release("a")
    b = m.admit("b")
    assert b == a and torch.equal(state[b], torch.zeros(3))
    views = m.views({0: torch.zeros((1, 1), dtype=torch.int32)})
    assert views[0].k_pages.shape == (9, 1, 4, 8) and views[1].state is state


def test_shared_cache_views():
    need = PagedKVNeed(2, 8)
    order = [RunEntry(0), RunEntry(1, cache_from=0), RunEntry(0)]
    m = manager([need, None, need], order)
    assert m.groups[0].entries == [0, 2]
    v = m.views({0: torch.zeros((1, 1), dtype=torch.int32)})
    assert v[1].k_pages.data_ptr() == v[0].k_pages.data_ptr() and not v[1].writable and v[0].writable
    assert v[2].k_pages.data_ptr() != v[0].k_pages.data_ptr()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    needs = [PagedKVNeed(1, 4), PagedKVNeed(1, 4, window=rng.choice([3, 9, 17])), PagedKVNeed(1, 4)]
    m = manager(needs, page=rng.choice([2, 4, 8]), pages=rng.choice([6, 12, 30]), slots=4)
    m.groups[0].kv = m.groups[1].kv = None
    live, n = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.can_admit():
            rid = f"r{n}"; n += 1
            m.admit(rid); live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(sorted(live))
            add = rng.choice([1, 1, 1, 2, 5, 11])
            short = m.pages_short(rid, live[rid], live[rid] + add)
            try:
                m.extend(rid, live[rid], live[rid] + add)
                assert short == 0
                live[rid] += add
                for g in m.groups:
                    t, first = g.tables[rid], g.first_needed_page(live[rid] - add)
                    assert len(t) == pages_for(live[rid], g.page_size)
                    assert all(p > 0 for p in t[first:]) and all(p == 0 for p in t[:first])
            except OutOfPages:
                assert short > 0
        elif live:
            rid = rng.choice(sorted(live))
            m.release(rid); del live[rid]
        m.check()
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(g.allocator.num_free == g.allocator.num_usable for g in m.groups)
    assert m.slots.num_free == 4
