"""A pool of page ids with a free list.

The reference hands out blocks from a counter that only grows and exits when
it runs out (src/examples/lib/inference_batch.cc:58-66); nothing is ever given
back.  Here pages return to the pool and are used again at once (the most
recently freed page is the next one handed out), so whether a page's contents
are valid is decided by the owning request's length, never by what the page
holds.
"""
from __future__ import annotations

from typing import List, Optional


class PageError(RuntimeError):
    """A page was freed twice, or one that is not held was freed."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() -> lowest id first
        self._held = bytearray(num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> Optional[List[int]]:
        """``n`` pages, or None (and nothing taken) if fewer are free."""
        if n < 0:
            raise ValueError("negative page count")
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = 1
        return out

    def free(self, pages) -> None:
        for p in pages:
            if p < 0 or p >= self.num_pages or not self._held[p]:
                raise PageError(f"page {p} is not held (double free?)")
            self._held[p] = 0
            self._free.append(p)

    def check(self) -> None:
        """Invariant: every page is either free exactly once or held."""
        seen = bytearray(self.num_pages)
        for p in self._free:
            if seen[p] or self._held[p]:
                raise PageError(f"page {p} is on the free list twice or also held")
            seen[p] = 1
        if sum(seen) + sum(self._held) != self.num_pages:
            raise PageError("a page is neither free nor held")
