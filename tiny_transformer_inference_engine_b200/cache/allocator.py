"""Hands out page ids (and state-slot ids) from a free list threaded through one array.

The contract is the one the reference's ``BlockAllocator`` keeps (serving/allocator.py:1-43;
tests/test_block_allocator.py:4-33): id 0 is scratch and never handed out (padding entries of
block tables point at it), the page freed last is the page handed out next, a request for
several pages is served whole or not at all, and a ``free`` that names a bad id changes nothing.

The form is this package's own: ``_link[p]`` holds, for a free page, the id of the free page
below it on the stack (``_END`` for the bottom one) and ``_HELD`` for a page that is handed
out, so one array answers "is it free" and "what comes next" and neither a Python list of free
ids nor a second flag array is kept.  Taking or returning a page moves ``_top`` and writes one
entry.
"""
from __future__ import annotations

from array import array
from typing import Iterable, List

_END, _HELD, _MARK = -1, -2, -3


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int, reserve_zero: bool = True):
        lowest = 1 if reserve_zero else 0
        if num_pages <= lowest:
            raise ValueError(f"a pool of {num_pages} pages has none to hand out (the first usable id is {lowest})")
        self.num_pages = int(num_pages)
        self._lowest = lowest
        # thread the stack so that ids come out ascending on first use: lowest on top, each linking to the next higher
        self._link = array("i", [_HELD] * lowest + [p + 1 for p in range(lowest, num_pages)])
        self._link[num_pages - 1] = _END
        self._top = lowest
        self._count = num_pages - lowest

    # ---------------------------------------------------------------- numbers
    @property
    def num_free(self) -> int:
        return self._count

    @property
    def num_usable(self) -> int:
        return self.num_pages - self._lowest

    def can_allocate(self, n: int) -> bool:
        return n <= self._count

    def is_free(self, p: int) -> bool:
        return self._link[p] != _HELD

    # ---------------------------------------------------------------- taking
    def allocate(self) -> int:
        p = self._top
        if p == _END:
            raise OutOfPages("the pool has no free page")
        self._top = self._link[p]
        self._link[p] = _HELD
        self._count -= 1
        return p

    def allocate_n(self, n: int) -> List[int]:
        if n > self._count:
            raise OutOfPages(f"{n} pages wanted, {self._count} free")
        return [self.allocate() for _ in range(n)]

    # ---------------------------------------------------------------- returning
    def free(self, pages: Iterable[int]) -> None:
        """Puts the pages back, the last one named on top.  Every id is checked first (inside the pool, handed out,
        named once); if one fails, the marks are undone and nothing has changed."""
        pages = [int(p) for p in pages]
        link, bad = self._link, None
        marked = 0
        for p in pages:
            if not self._lowest <= p < self.num_pages:
                bad = f"page id {p} is outside {self._lowest}..{self.num_pages - 1}"
            elif link[p] == _MARK:
                bad = f"page {p} is named twice in one free"
            elif link[p] != _HELD:
                bad = f"page {p} is free already"
            if bad:
                break
            link[p] = _MARK                                   # a held page seen once
            marked += 1
        if bad:
            for p in pages[:marked]:
                link[p] = _HELD
            raise ValueError(bad)
        for p in pages:
            link[p] = self._top
            self._top = p
        self._count += len(pages)
