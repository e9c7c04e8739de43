"""The cache manager: paged keys and values with a block table per request, in groups,
and slots for per-request state of fixed size.

The reference keeps one pool ``kv[L, 2, pages, page, Hkv, D]`` with one allocator and a
Python block table per ``Sequence`` (serving/kv_pool.py:12-21, serving/sequence.py:14-30).
Here the cache needs of a model's run entries (an entry may have several: a block
reports one per cache-using sub-part) are sorted into **groups** by what they ask for
(kv heads, head size, window, page size): a group has its own page size, its own number
of pages, its own allocator and its own block table per request, so a windowed layer
can give pages back - and needs far fewer pages to begin with - while a full-attention
layer keeps all of its.  A page id addresses the same slab in every cache layer of its
group and in K and V, as in the reference.

Sizing.  With an explicit ``num_pages`` every group gets room for the same number of
tokens (``(num_pages - 1) * page_size``; a group with another page size gets as many
pages of its own size as that takes).  With a byte budget the manager looks for the
largest number of tokens T such that all groups together fit the budget, where a
windowed group never needs more than ``max_slots`` requests x (window + longest
step) tokens: its share stops growing there and the rest goes to the other groups.

Pages go back to the allocator when the request is released (finished or preempted)
and, for a windowed group, as soon as every position of the page lies before the
window of the next token to run; a freed page's table entry becomes 0 (scratch) and is
never read because the kernels start at the window's first key.  Freed pages are used
again at once (LIFO) and are not cleared: reads are bounded by the request's length.

State slots: ``max_slots`` ids; a request takes one at admission and gives it back at
release.  A need of ``FixedStateNeed`` gets a tensor ``[max_slots + 1, *shape]`` whose
row ``slot`` is zeroed when the slot is handed out; the last row is scratch (slot id -1,
the padding rows of a captured decode step, indexes it).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Tuple

import torch

from .allocator import PageAllocator, OutOfPages
from ..parts.base import PagedKVNeed, FixedStateNeed, PagedKVView, FixedStateView, RunEntry

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def pages_for(num_tokens: int, page_size: int) -> int:
    return -(-num_tokens // page_size)            # serving/sequence.py:32-33


def _as_list(need) -> list:
    if need is None:
        return []
    return list(need) if isinstance(need, (list, tuple)) else [need]


@dataclass
class CacheGroup:
    need: PagedKVNeed
    page_size: int
    num_pages: int
    entries: List[Tuple[int, int]] = field(default_factory=list)   # (run entry, index of the need in it), in cache-layer order
    allocator: PageAllocator = None
    kv: Optional[torch.Tensor] = None                         # [layers, 2, pages, Hkv, page, D]
    tables: Dict[Hashable, List[int]] = field(default_factory=dict)

    @property
    def window(self):
        return self.need.window

    def first_needed_page(self, start: int) -> int:
        """First logical page a token at position >= start can still read."""
        if self.window is None:
            return 0
        first_key = max(0, start - self.window + 1)
        return first_key // self.page_size

    def bytes_per_page(self, elem_size: int) -> int:
        # models/model_config.py:84-88, per group
        return 2 * len(self.entries) * self.page_size * self.need.num_kv_heads * self.need.head_dim * elem_size

    def pages_of_request(self, num_tokens: int, max_step_tokens: Optional[int]) -> int:
        """The most pages a request of ``num_tokens`` holds at one time: all of them, or - with a window - those
        of the window plus the longest step (pages the window has passed are given back before new ones are taken)."""
        whole = pages_for(num_tokens, self.page_size)
        if self.window is None or max_step_tokens is None:
            return whole
        return min(whole, pages_for(self.window + max_step_tokens - 1, self.page_size) + 1)


class CacheManager:
    def __init__(self, needs: List[object], run_order: List[RunEntry], page_size: int,
                 num_pages: Optional[int], max_slots: int, dtype: str, device,
                 kv_budget_bytes: Optional[int] = None, allocate: bool = True, max_step_tokens: Optional[int] = None):
        """``needs[e]``: what run entry ``e`` asks for - None, one need, or a list of needs.  ``page_size`` is the
        page size of every need that names none.  ``max_step_tokens``: the most tokens a request brings in one
        step (the scheduler's budget); it bounds what a windowed group has to hold."""
        self.default_page_size, self.max_slots = int(page_size), int(max_slots)
        self.max_step_tokens = max_step_tokens
        self.dtype = _TORCH_DTYPES[dtype]
        self.device = torch.device(device)
        self.run_order = list(run_order)
        self.groups: List[CacheGroup] = []
        self.entry_needs: List[list] = [_as_list(n) for n in needs]
        self.entry_group: Dict[Tuple[int, int], Tuple[int, int]] = {}    # (run entry, need index) -> (group, cache layer)
        self.entry_state: Dict[Tuple[int, int], torch.Tensor] = {}
        self._state_needs: Dict[Tuple[int, int], FixedStateNeed] = {}
        by_need: Dict[PagedKVNeed, int] = {}
        for e, entry_needs in enumerate(self.entry_needs):
            for k, need in enumerate(entry_needs):
                if isinstance(need, PagedKVNeed):
                    if need not in by_need:
                        by_need[need] = len(self.groups)
                        ps = int(need.page_size or self.default_page_size)
                        if ps < 1:
                            raise ValueError(f"run entry {e}: page size {ps}")
                        self.groups.append(CacheGroup(need, ps, 0))
                    g = by_need[need]
                    self.entry_group[(e, k)] = (g, len(self.groups[g].entries))
                    self.groups[g].entries.append((e, k))
                elif isinstance(need, FixedStateNeed):
                    self._state_needs[(e, k)] = need
                else:
                    raise TypeError(f"run entry {e}: unknown cache need {need!r}")
        elem = torch.empty((), dtype=self.dtype).element_size()
        if num_pages is not None:
            tokens = (int(num_pages) - 1) * self.default_page_size
            counts = [pages_for(tokens, g.page_size) + 1 for g in self.groups]
        else:
            counts = self._size_from_budget(int(kv_budget_bytes or 0), elem)
        for g, n in zip(self.groups, counts):
            g.num_pages = max(2, int(n))
            g.allocator = PageAllocator(g.num_pages)
            if allocate:
                # zero-initialised like the reference's pool (serving/kv_pool.py:12-16)
                g.kv = torch.zeros((len(g.entries), 2, g.num_pages, g.need.num_kv_heads, g.page_size,
                                    g.need.head_dim), dtype=self.dtype, device=self.device)
        self.slots = PageAllocator(self.max_slots, reserve_zero=False)
        self.slot_of: Dict[Hashable, int] = {}
        if allocate:
            for key, need in self._state_needs.items():
                self.entry_state[key] = torch.zeros((self.max_slots + 1, *need.shape), dtype=_TORCH_DTYPES[need.dtype],
                                                    device=self.device)

    def _size_from_budget(self, budget: int, elem: int) -> List[int]:
        """Pages per group (scratch page included) for the largest token capacity that fits ``budget`` bytes."""
        def pages(g: CacheGroup, tokens: int) -> int:
            n = pages_for(tokens, g.page_size)
            if g.window is not None and self.max_step_tokens is not None:
                n = min(n, self.max_slots * g.pages_of_request(tokens, self.max_step_tokens))
            return n + 1

        def cost(tokens: int) -> int:
            return sum(pages(g, tokens) * g.bytes_per_page(elem) for g in self.groups)

        lo, hi = 0, 1
        while cost(hi) <= budget and hi < (1 << 40):
            lo, hi = hi, hi * 2
        while hi - lo > 1:                                     # cost is monotone in tokens
            mid = (lo + hi) // 2
            lo, hi = (mid, hi) if cost(mid) <= budget else (lo, mid)
        return [pages(g, lo) for g in self.groups]

    # ---------------------------------------------------------------- requests
    def has_request(self, rid) -> bool:
        return rid in self.slot_of

    def can_admit(self) -> bool:
        return self.slots.num_free > 0

    def admit(self, rid) -> int:
        """Gives the request a state slot and empty block tables."""
        if rid in self.slot_of:
            raise ValueError(f"request {rid!r} is already admitted")
        slot = self.slots.allocate()
        self.slot_of[rid] = slot
        for g in self.groups:
            g.tables[rid] = []
        for state in self.entry_state.values():
            state[slot].zero_()
        return slot
    def _plan(self, rid, start: int, new_len: int):
        """Per group: (pages to free now, logical pages to fill)."""
        plan = []
        for g in self.groups:
            table = g.tables[rid]
            last = pages_for(new_len, g.page_size)
            if g.window is None:                               # nothing is ever given back early: only growth
                plan.append(([], list(range(len(table), last)), last))
                continue
            first = g.first_needed_page(start)
            to_free = [(i, p) for i, p in enumerate(table[:first]) if p != 0]
            to_fill = [i for i in range(first, last) if i >= len(table) or table[i] == 0]
            plan.append((to_free, to_fill, last))
        return plan

    def pages_short(self, rid, start: int, new_len: int) -> int:
        """How many pages are lacking (max over groups) to hold positions < new_len, counting
        pages that a window lets go first.  0 means ``extend`` will succeed."""
        short = 0
        for g, (to_free, to_fill, _) in zip(self.groups, self._plan(rid, start, new_len)):
            short = max(short, len(to_fill) - len(to_free) - g.allocator.num_free)
        return max(0, short)

    def extend(self, rid, start: int, new_len: int) -> None:
        """Makes room for tokens at positions ``start .. new_len-1`` in every group, after
        giving back pages that no token at a position >= start can read.  All or nothing
        as far as new pages go: raises OutOfPages and allocates none if any group is short."""
        if rid not in self.slot_of:
            raise KeyError(f"request {rid!r} is not admitted")
        if not 0 <= start <= new_len:
            raise ValueError(f"bad span start={start} new_len={new_len}")
        plan = self._plan(rid, start, new_len)
        for g, (to_free, _, _) in zip(self.groups, plan):
            if to_free:
                g.allocator.free([p for _, p in to_free])
                for i, _ in to_free:
                    g.tables[rid][i] = 0
        for g, (_, to_fill, _) in zip(self.groups, plan):
            if not g.allocator.can_allocate(len(to_fill)):
                raise OutOfPages(f"need {len(to_fill)} pages, only {g.allocator.num_free} free")
        for g, (_, to_fill, last) in zip(self.groups, plan):
            table = g.tables[rid]
            if len(table) < last:
                table.extend([0] * (last - len(table)))
            for i, p in zip(to_fill, g.allocator.allocate_n(len(to_fill))):
                table[i] = p

    def release(self, rid) -> None:
        """Gives back every page and the state slot of the request."""
        if rid not in self.slot_of:
            raise KeyError(f"request {rid!r} is not admitted")
        for g in self.groups:
            g.allocator.free([p for p in g.tables[rid] if p != 0])
            del g.tables[rid]
        self.slots.free([self.slot_of.pop(rid)])

    # ---------------------------------------------------------------- numbers
    @property
    def num_free_pages(self) -> int:
        return min((g.allocator.num_free for g in self.groups), default=0)

    @property
    def num_usable_pages(self) -> int:
        return min((g.allocator.num_usable for g in self.groups), default=0)

    @property
    def page_size(self) -> int:
        """The smallest page size in use: a portion cut at a multiple of it ends on a page edge in that group."""
        return min((g.page_size for g in self.groups), default=self.default_page_size)

    def request_fits_empty_pool(self, num_tokens: int) -> bool:
        """Whether a lone request of ``num_tokens`` could be held with every other page free."""
        return all(g.pages_of_request(num_tokens, self.max_step_tokens) <= g.allocator.num_usable for g in self.groups)

    def admission_headroom(self, num_tokens: int, reserve: int) -> bool:
        """The reference's admission rule, group by group (serving/scheduler.py:33-37): after the pages of a request
        of ``num_tokens`` are taken, ``reserve`` pages must be left."""
        return all(g.allocator.num_free - g.pages_of_request(num_tokens, self.max_step_tokens) >= reserve for g in self.groups)

    def table(self, group: int, rid) -> List[int]:
        return self.groups[group].tables[rid]

    def check(self) -> None:
        """Every page is free or held by exactly one request; no slot is held twice."""
        for gi, g in enumerate(self.groups):
            held = {}
            for rid, table in g.tables.items():
                for p in table:
                    if p == 0:
                        continue
                    if p in held:
                        raise AssertionError(f"group {gi}: page {p} held by {held[p]!r} and {rid!r}")
                    if g.allocator.is_free(p):
                        raise AssertionError(f"group {gi}: page {p} of {rid!r} is on the free list")
                    held[p] = rid
            if len(held) + g.allocator.num_free != g.allocator.num_usable:
                raise AssertionError(f"group {gi}: {g.allocator.num_usable - len(held) - g.allocator.num_free} page(s) lost")
        if len(set(self.slot_of.values())) != len(self.slot_of):
            raise AssertionError("a state slot is held twice")
        if len(self.slot_of) + self.slots.num_free != self.max_slots:
            raise AssertionError("a state slot is lost")

    # ---------------------------------------------------------------- views for a step
    def views(self, block_tables: Dict[int, torch.Tensor]) -> List[List[object]]:
        """For every run entry the list of its cache views, one per need in the order the block reported them, for
        a step whose per-group block tables (device, int32 [N, max_pages]) are given.  An entry that reads another
        entry's cache gets that entry's views, not writable."""
        views: List[List[object]] = []
        for e, entry in enumerate(self.run_order):
            src = e if entry.cache_from is None else entry.cache_from
            writable = entry.cache_from is None
            mine = []
            for k in range(len(self.entry_needs[src])):
                if (src, k) in self.entry_group:
                    gi, layer = self.entry_group[(src, k)]
                    g = self.groups[gi]
                    mine.append(PagedKVView(g.kv[layer, 0], g.kv[layer, 1], block_tables[gi], g.page_size, writable))
                else:
                    mine.append(FixedStateView(self.entry_state[(src, k)], writable))
            views.append(mine)
        return views
