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
    assert len(m.groups) == 2 and m.groups[0].entries == [(0, 0), (2, 0)] and m.groups[1].entries == [(1, 0)]
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
    state = m.entry_state[(1, 0)]
    assert state.shape == (3, 3)                                   # two slots and the scratch row that slot id -1 indexes
    a = m.admit("a")
    state[a] += 5
    m.release("a")
    b = m.admit("b")
    assert b == a and torch.equal(state[b], torch.zeros(3))
    views = m.views({0: torch.zeros((1, 1), dtype=torch.int32)})
    assert views[0][0].k_pages.shape == (9, 1, 4, 8) and views[1][0].state is state


def test_shared_cache_views():
    need = PagedKVNeed(2, 8)
    order = [RunEntry(0), RunEntry(1, cache_from=0), RunEntry(0)]
    m = manager([need, None, need], order)
    assert m.groups[0].entries == [(0, 0), (2, 0)]
    v = [x[0] for x in m.views({0: torch.zeros((1, 1), dtype=torch.int32)})]
    assert v[1].k_pages.data_ptr() == v[0].k_pages.data_ptr() and not v[1].writable and v[0].writable
    assert v[2].k_pages.data_ptr() != v[0].k_pages.data_ptr()


def test_an_entry_with_several_needs_gets_as_many_views():
    """A block whose mixer keeps pages and a state of fixed size, beside a plain one: the views come in the order
    of the needs, the pages of both entries share a group, and a reader of the first entry sees both views."""
    kv = PagedKVNeed(1, 8)
    order = [RunEntry(0), RunEntry(1), RunEntry(2, cache_from=0)]
    m = manager([[kv, FixedStateNeed((5,)), FixedStateNeed((2, 2), "bfloat16")], kv, []], order, slots=2)
    assert m.groups[0].entries == [(0, 0), (1, 0)] and sorted(m.entry_state) == [(0, 1), (0, 2)]
    v = m.views({0: torch.zeros((1, 1), dtype=torch.int32)})
    assert [type(x).__name__ for x in v[0]] == ["PagedKVView", "FixedStateView", "FixedStateView"]
    assert v[0][1].state.shape == (3, 5) and v[0][2].state.shape == (3, 2, 2) and v[0][2].state.dtype == torch.bfloat16
    assert len(v[1]) == 1 and len(v[2]) == 3 and not any(x.writable for x in v[2])
    assert v[2][1].state is v[0][1].state
    a = m.admit("a")
    v[0][1].state[a] += 1
    m.release("a")
    assert m.admit("b") == a and float(v[0][1].state[a].abs().sum()) == 0


def test_each_group_has_its_own_page_size_and_page_count():
    """An explicit page count gives every group room for the same number of tokens in pages of its own size; a byte
    budget stops growing a windowed group where its requests can hold no more and spends the rest on the others."""
    full, win, big = PagedKVNeed(1, 8), PagedKVNeed(1, 8, window=6), PagedKVNeed(2, 16, page_size=16)
    m = manager([full, win, big], page=4, pages=9)                 # 8 usable pages of 4 tokens = 32 tokens
    assert [g.page_size for g in m.groups] == [4, 4, 16] and [g.num_pages for g in m.groups] == [9, 9, 3]
    assert m.groups[2].kv.shape == (1, 2, 3, 2, 16, 16) and m.page_size == 4
    m.admit("a"); m.extend("a", 0, 17)
    assert m.table(0, "a") == [1, 2, 3, 4, 5] and m.table(2, "a") == [1, 2]
    with pytest.raises(OutOfPages):
        m.extend("a", 17, 33)                                      # 33 tokens: 9 pages of 4, 3 of 16
    assert m.table(0, "a") == [1, 2, 3, 4, 5] and m.table(2, "a") == [1, 2]
    m.release("a"); m.check()
    # a byte budget: float32, group "full": 2*1*4*1*8*4 = 256 B/page, "win" the same
    order = [RunEntry(0), RunEntry(1)]
    mb = CacheManager([full, win], order, 4, None, 2, "float32", "cpu", kv_budget_bytes=256 * 60, allocate=False,
                      max_step_tokens=8)
    # a windowed request holds at most pages_for(6 + 8 - 1, 4) + 1 = 5 pages; two slots: 10 pages (+ scratch)
    assert mb.groups[1].num_pages == 11 and mb.groups[0].num_pages == 60 - 11
    assert mb.request_fits_empty_pool(48 * 4) and not mb.request_fits_empty_pool(48 * 4 + 1)
    assert mb.admission_headroom(40 * 4, 5) and not mb.admission_headroom(40 * 4, 6)    # the windowed group: 10 free - 5
    # without a bound on the step the windowed group is sized like the other
    mu = CacheManager([full, win], order, 4, None, 2, "float32", "cpu", kv_budget_bytes=256 * 60, allocate=False)
    assert [g.num_pages for g in mu.groups] == [30, 30]


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
