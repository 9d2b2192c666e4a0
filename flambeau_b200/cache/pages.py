"""The page allocator: a fixed number of page ids, handed out and taken back.

Free pages are reused in the order they were returned (first in, first out),
like the reference's host allocator (crates/forward/src/core/scratch.rs:602-703).
A request for several pages is all-or-nothing.
"""
from __future__ import annotations

from collections import deque


class PageError(RuntimeError):
    pass


class OutOfPages(PageError):
    def __init__(self, wanted: int, free: int, total: int):
        super().__init__(f"{wanted} cache pages wanted, {free} of {total} free")
        self.wanted, self.free, self.total = wanted, free, total


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = int(n_pages)
        self._free = deque(range(self.n_pages))
        self._held = [False] * self.n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def take(self, count: int) -> list:
        """`count` page ids, or OutOfPages with nothing taken."""
        if count < 0:
            raise ValueError("negative page count")
        if count > len(self._free):
            raise OutOfPages(count, len(self._free), self.n_pages)
        out = [self._free.popleft() for _ in range(count)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages:
                raise PageError(f"page id {p} is outside the pool of {self.n_pages}")
            if not self._held[p]:
                raise PageError(f"page {p} is given back but is not held")
            self._held[p] = False
            self._free.append(p)

    def is_held(self, page: int) -> bool:
        return self._held[page]
