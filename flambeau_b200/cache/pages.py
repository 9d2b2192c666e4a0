"""The page books of the cache manager, kept by the C++ host code of the kernel library
(`csrc/host_cache.cpp`): page pools, per-request page lists and lengths, reservation and release.

Free pages are reused in the order they were returned (first in, first out), like the reference's host
allocator (crates/forward/src/core/scratch.rs:602-703).  A request for several pages is all-or-nothing.
This module is the thin Python face of those books: errors become exceptions, ids become lists.
"""
from __future__ import annotations

import ctypes

import numpy as np

from ..kernels.library import lib


class PageError(RuntimeError):
    pass


class OutOfPages(PageError):
    def __init__(self, wanted: int, free: int, total: int, message: str | None = None):
        super().__init__(message or f"{wanted} cache pages wanted, {free} of {total} free")
        self.wanted, self.free, self.total = wanted, free, total


ERR_PAGES, ERR_STATE, ERR_LIMIT, ERR_BATCH = -10, -11, -12, -13


def _ints(values) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.int32)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


class Books:
    """One cache's books: `n_pages[g]` pages and window `windows[g]` (0 = none) for each group g."""

    def __init__(self, n_pages: list, windows: list, page_size: int, max_requests: int, max_pages_per_request: int):
        if any(n <= 0 for n in n_pages):
            raise ValueError("a page pool needs at least one page")
        self._lib = lib()
        self.n_groups = len(n_pages)
        self._scratch = np.zeros(max(self.n_groups, 1), dtype=np.int32)
        self._h = self._lib.fbh_cache_new(self.n_groups, _ptr(_ints(n_pages if n_pages else [0])),
                                          _ptr(_ints(windows if windows else [0])), int(page_size), int(max_requests),
                                          int(max_pages_per_request))
        if not self._h:
            raise PageError(self._message())

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.fbh_cache_free(h)

    # ---- errors ----
    def _message(self) -> str:
        return self._lib.fbh_last_error().decode(errors="replace")

    def _raise(self, code: int):
        msg = self._message()
        if code == ERR_PAGES:
            nums = [int(t) for t in msg.replace(",", " ").split() if t.isdigit()]
            raise OutOfPages(*(nums[:3] if len(nums) >= 3 else (0, 0, 0)), message=msg)
        raise PageError(msg)

    def _ok(self, code: int) -> int:
        if code < 0:
            self._raise(code)
        return code

    # ---- requests ----
    def has_slot(self) -> bool:
        return bool(self._lib.fbh_has_slot(self._h))

    def admit(self) -> int:
        return self._ok(self._lib.fbh_admit(self._h))

    def admit_at(self, length: int, first_pages) -> int:
        """A slot for a request of `length` tokens whose group g holds its pages from first_pages[g] on."""
        fp = _ints(first_pages if len(first_pages) else [0])
        return self._ok(self._lib.fbh_admit_at(self._h, int(length), _ptr(fp)))

    def release(self, slot: int) -> None:
        self._ok(self._lib.fbh_release(self._h, slot))

    def length(self, slot: int) -> int:
        return self._ok(self._lib.fbh_length(self._h, slot))

    def reserved_to(self, slot: int) -> int:
        return self._ok(self._lib.fbh_reserved_to(self._h, slot))

    def free_pages(self) -> list:
        self._lib.fbh_free_pages(self._h, _ptr(self._scratch))
        return self._scratch[:self.n_groups].tolist()

    def pool_pages(self, group: int) -> int:
        return self._lib.fbh_pool_pages(self._h, group)

    def is_held(self, group: int, page: int) -> bool:
        return bool(self._lib.fbh_is_held(self._h, group, page))

    def pages_needed(self, slot: int, n_new: int) -> list:
        self._ok(self._lib.fbh_pages_needed(self._h, slot, int(n_new), _ptr(self._scratch)))
        return self._scratch[:self.n_groups].tolist()

    def reserve_all(self, slots, n_new, dry_run: bool = False) -> bool:
        """Pages for n_new[i] more tokens of every slots[i], or none at all.  dry_run: only whether they fit."""
        s, k = _ints(slots), _ints(n_new)
        code = self._lib.fbh_reserve_all(self._h, len(s), _ptr(s), _ptr(k), 1 if dry_run else 0)
        if dry_run and code == ERR_PAGES:
            return False
        self._ok(code)
        return True

    def commit(self, slots, n_new) -> None:
        s, k = _ints(slots), _ints(n_new)
        self._ok(self._lib.fbh_commit(self._h, len(s), _ptr(s), _ptr(k)))

    def pages(self, slot: int, group: int) -> list:
        n = self._ok(self._lib.fbh_pages(self._h, slot, group, None, 0))
        out = np.empty(max(n, 1), dtype=np.int32)
        self._ok(self._lib.fbh_pages(self._h, slot, group, _ptr(out), n))
        return out[:n].tolist()

    def first_live_page(self, slot: int, group: int) -> int:
        return self._ok(self._lib.fbh_first_live_page(self._h, slot, group))

    def n_pages_of(self, slot: int, group: int) -> int:
        return self._ok(self._lib.fbh_pages(self._h, slot, group, None, 0))

    def check_invariants(self) -> None:
        self._ok(self._lib.fbh_check_invariants(self._h))

    @property
    def handle(self):
        return self._h
