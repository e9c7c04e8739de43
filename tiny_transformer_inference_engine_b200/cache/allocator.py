"""Hands out page ids (and state-slot ids).

Same contract as the reference's ``BlockAllocator`` (serving/allocator.py:1-43): id 0
is scratch and never handed out (padding entries of block tables point at it), free
ids form a LIFO stack so a freed page is the next one used, ``allocate_n`` is all or
nothing, and ``free`` checks every id (range, double free, duplicates) before it
changes anything.
"""
from __future__ import annotations

from typing import Iterable, List


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int, reserve_zero: bool = True):
        first = 1 if reserve_zero else 0
        if num_pages < first + 1:
            raise ValueError(f"need at least {first + 1} pages, got {num_pages}")
        self.num_pages = num_pages
        self._first = first
        self._free: List[int] = list(range(num_pages - 1, first - 1, -1))
        self._is_free = [False] * first + [True] * (num_pages - first)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_usable(self) -> int:
        return self.num_pages - self._first

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("out of pages")
        p = self._free.pop()
        self._is_free[p] = False
        return p

    def allocate_n(self, n: int) -> List[int]:
        if not self.can_allocate(n):
            raise OutOfPages(f"need {n} pages, only {self.num_free} free")
        return [self.allocate() for _ in range(n)]

    def free(self, pages: Iterable[int]) -> None:
        pages = list(pages)
        seen = set()
        for p in pages:
            if not (self._first <= p < self.num_pages):
                raise ValueError(f"invalid page id {p}")
            if self._is_free[p] or p in seen:
                raise ValueError(f"double free of page {p}")
            seen.add(p)
        for p in pages:
            self._is_free[p] = True
            self._free.append(p)

    def is_free(self, p: int) -> bool:
        return self._is_free[p]
