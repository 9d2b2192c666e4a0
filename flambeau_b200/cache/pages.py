"""The page allocator: a fixed number of page ids, handed out and taken back.

Free pages are reused in the order they were returned (first in, first out),
like the reference's host allocator (crates/forward/src/core/scratch.rs:602-703).
A request for several pages is all-or-nothing.
"""
from __future__ import annotations

from collections import deque

import numpy as np


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


class PageList:
    """The physical pages of one request in one group, by logical page index (-1 = given back), kept in a
    numpy array so that a block-table row is one memory copy."""
    __slots__ = ("arr", "n", "first_live")

    def __init__(self, capacity: int = 16):
        self.arr = np.full(max(capacity, 1), -1, dtype=np.int32)
        self.n = 0
        self.first_live = 0              # logical pages below this index have been given back

    def __len__(self) -> int:
        return self.n

    def __iter__(self):
        return iter(self.arr[:self.n].tolist())

    def __getitem__(self, i):
        return self.arr[:self.n][i]

    def extend(self, pages) -> None:
        k = len(pages)
        if self.n + k > self.arr.size:
            grown = np.full(max(2 * self.arr.size, self.n + k), -1, dtype=np.int32)
            grown[:self.n] = self.arr[:self.n]
            self.arr = grown
        self.arr[self.n:self.n + k] = pages
        self.n += k

    def give_back_prefix(self, upto: int) -> list:
        """Mark logical pages [first_live, upto) as given back and return their ids."""
        upto = min(upto, self.n)
        if upto <= self.first_live:
            return []
        back = self.arr[self.first_live:upto]
        out = back[back >= 0].tolist()
        self.arr[self.first_live:upto] = -1
        self.first_live = upto
        return out

    def live(self) -> list:
        a = self.arr[self.first_live:self.n]
        return a[a >= 0].tolist()

    def view(self) -> np.ndarray:
        return self.arr[:self.n]
