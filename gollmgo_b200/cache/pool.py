"""Fixed pool of cache pages with a free list and reference counts.

Same semantics as the reference's BlockPool (internal/kvcache/block_pool.go:19-86):
``allocate(n)`` gives n pages or raises without taking any, a page goes back to
the free list when its count reaches zero, and the free list is last-in-first-out
so that a page given back is the next one handed out (replays reproduce page ids).
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than were asked for."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() gives page 0 first
        self._refs = [0] * num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def utilization(self) -> float:
        return self.num_used / self.num_pages

    def allocate(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"asked for {n} pages, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._refs[p] = 1
        self.high_water = max(self.high_water, self.num_used)
        return pages

    def ref(self, page: int) -> None:
        if self._refs[page] <= 0:
            raise RuntimeError(f"page {page} is free; cannot share it")
        self._refs[page] += 1

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise RuntimeError(f"page {page} is not of this pool")
        if self._refs[page] <= 0:
            raise RuntimeError(f"page {page} freed twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def free_pages(self) -> List[int]:
        return list(self._free)
