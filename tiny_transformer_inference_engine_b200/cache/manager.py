"""The cache manager: paged keys and values with a block table per request, in groups,
and slots for per-request state of fixed size.

The reference keeps one pool ``kv[L, 2, pages, page, Hkv, D]`` with one allocator and a
Python block table per ``Sequence`` (serving/kv_pool.py:12-21, serving/sequence.py:14-30).
Here the run entries of a model that need a cache are sorted into **groups** by what
they need (kv heads, head size, window): a group has its own pages, its own allocator
and its own block table per request, so a windowed layer can give pages back while a
full-attention layer keeps all of its.  A page id addresses the same slab in every
cache layer of its group and in K and V, as in the reference.

Pages go back to the allocator when the request is released (finished or preempted)
and, for a windowed group, as soon as every position of the page lies before the
window of the next token to run; a freed page's table entry becomes 0 (scratch) and is
never read because the kernels start at the window's first key.  Freed pages are used
again at once (LIFO) and are not cleared: reads are bounded by the request's length.

State slots: ``max_slots`` ids; a request takes one at admission and gives it back at
release.  A run entry that asks for ``FixedStateNeed`` gets a tensor
``[max_slots, *shape]`` whose row ``slot`` is zeroed when the slot is handed out.
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


@dataclass
class CacheGroup:
    need: PagedKVNeed
    page_size: int
    num_pages: int
    entries: List[int] = field(default_factory=list)          # run entries, in cache-layer order
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


class CacheManager:
    def __init__(self, needs: List[Optional[object]], run_order: List[RunEntry], page_size: int,
                 num_pages: Optional[int], max_slots: int, dtype: str, device,
                 kv_budget_bytes: Optional[int] = None, allocate: bool = True):
        self.page_size, self.max_slots = int(page_size), int(max_slots)
        self.dtype = _TORCH_DTYPES[dtype]
        self.device = torch.device(device)
        self.run_order = list(run_order)
        self.groups: List[CacheGroup] = []
        self.entry_group: Dict[int, Tuple[int, int]] = {}      # run entry -> (group, cache layer)
        self.entry_state: Dict[int, torch.Tensor] = {}
        self._state_needs: Dict[int, FixedStateNeed] = {}
        by_need: Dict[PagedKVNeed, int] = {}
        for e, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, PagedKVNeed):
                if need not in by_need:
                    by_need[need] = len(self.groups)
                    self.groups.append(CacheGroup(need, self.page_size, 0))
                g = by_need[need]
                self.entry_group[e] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(e)
            elif isinstance(need, FixedStateNeed):
                self._state_needs[e] = need
            else:
                raise TypeError(f"run entry {e}: unknown cache need {need!r}")
        elem = torch.empty((), dtype=self.dtype).element_size()
        if num_pages is None:
            per_page = sum(g.bytes_per_page(elem) for g in self.groups) or 1
            num_pages = max(2, int(kv_budget_bytes or 0) // per_page)
        for g in self.groups:
            g.num_pages = int(num_pages)
            g.allocator = PageAllocator(g.num_pages)
            if allocate:
                # zero-initialised like the reference's pool (serving/kv_pool.py:12-16)
                g.kv = torch.zeros((len(g.entries), 2, g.num_pages, g.need.num_kv_heads, self.page_size,
                                    g.need.head_dim), dtype=self.dtype, device=self.device)
        self.slots = PageAllocator(self.max_slots, reserve_zero=False)
        self.slot_of: Dict[Hashable, int] = {}
        if allocate:
            for e, need in self._state_needs.items():
                self.entry_state[e] = torch.zeros((self.max_slots, *need.shape), dtype=_TORCH_DTYPES[need.dtype],
                                                  device=self.device)

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

    def max_tokens_in_empty_pool(self) -> int:
        return self.num_usable_pages * self.page_size

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
    def views(self, block_tables: Dict[int, torch.Tensor]) -> List[object]:
        """One cache view per run entry for a step whose per-group block tables (device,
        int32 [N, max_pages]) are given."""
        views: List[object] = []
        for e, entry in enumerate(self.run_order):
            src = e if entry.cache_from is None else entry.cache_from
            writable = entry.cache_from is None
            if src in self.entry_group:
                gi, layer = self.entry_group[src]
                g = self.groups[gi]
                views.append(PagedKVView(g.kv[layer, 0], g.kv[layer, 1], block_tables[gi], g.page_size, writable))
            elif src in self.entry_state:
                views.append(FixedStateView(self.entry_state[src], writable))
            else:
                views.append(None)
        return views
