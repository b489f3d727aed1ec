"""Page and slot pools: plain host bookkeeping, no device memory.

The reference's ``BlockPool`` is a LIFO free list with reference counts
(``pkg/inference/paged_kvcache.go:34-117``).  Pages here have one owner at a time, so the
pool tracks ownership instead of counts and refuses a page that is freed twice.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """The pool cannot give as many pages as were asked for; nothing was taken."""


class OutOfSlots(RuntimeError):
    """Every per-request state slot is in use."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() gives page 0 first
        self._held = [False] * num_pages

    @property
    def free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        """``n`` pages, all or none."""
        if n > len(self._free):
            raise OutOfPages(f"asked for {n} pages, {len(self._free)} of {self.num_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise ValueError(f"page {page} is not of this pool (0..{self.num_pages - 1})")
        if not self._held[page]:
            raise RuntimeError(f"page {page} freed twice")
        self._held[page] = False
        self._free.append(page)

    def held_pages(self) -> List[int]:
        return [p for p, h in enumerate(self._held) if h]


class SlotPool(PagePool):
    """Ids of the fixed-size per-request state slots."""

    def take_one(self) -> int:
        try:
            return self.take(1)[0]
        except OutOfPages:
            raise OutOfSlots(f"all {self.num_pages} request slots are in use") from None
