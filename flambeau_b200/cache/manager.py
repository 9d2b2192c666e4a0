"""The cache manager: paged keys and values per group of layers, a block table
per request and group, and slots of fixed-size state per request.

Layers whose mixers need the same cache geometry (key/value heads, head size,
window) form a group.  A group has one page-id space: page p of a request is
row p of every layer's pool in the group, so pages are taken once per request
and step, not once per layer (the reference keeps one allocator per layer,
crates/forward/src/core/scratch.rs:438-463, 602-703).  Groups with different
needs have pools, tables and release rules of their own.

Pages are taken before a step for every new token of the step (all or
nothing), and given back
  * when a request ends, and
  * in a group with a window W, after the step that makes them dead: a page
    whose last position is below `length - W + 1` can be seen by no future
    query (every future query sits at p >= length and sees [p-W+1, p]).
The reference bounds windowed layers with ring slabs instead and rejects paged
windowed attention (crates/forward/src/core/composites/standard_attn.rs:436-441).

The manager, not the caller, owns each request's length.  The books themselves (pools, page lists, lengths,
reservation, release, invariants) are kept by the C++ host code of the kernel library (`csrc/host_cache.cpp`,
reached through `cache.pages.Books`); this module owns the device tensors, the grouping of layers and the
request ids.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..parts.base import KVRequirement, StateRequirement
from .pages import Books, OutOfPages, PageError


@dataclass
class CallPlan:
    """What one entry of the model's run order needs from the cache."""
    kv: Optional[KVRequirement] = None        # None: the mixer keeps no keys/values
    state: Optional[StateRequirement] = None
    cache_from: Optional[int] = None          # read the cache owned by that earlier call


@dataclass
class LayerCacheView:
    """What a mixer sees of the cache during one call."""
    k_pool: Optional[torch.Tensor]
    v_pool: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]       # device int32 [sequences of the step, table columns]: live pages only
    table_base: Optional[torch.Tensor] = None # device int32 [sequences]: the logical page column 0 stands for
    page_size: int = 16
    writable: bool = False
    group: int = -1
    state: Optional[torch.Tensor] = None      # [slots, *shape] for mixers with fixed-size state


class PageView:
    """The physical pages of one request in one group, by logical page index (-1 = given back)."""
    __slots__ = ("_books", "_slot", "_group")

    def __init__(self, books: Books, slot: int, group: int):
        self._books, self._slot, self._group = books, slot, group

    def __len__(self) -> int:
        return self._books.n_pages_of(self._slot, self._group)

    def __iter__(self):
        return iter(self._books.pages(self._slot, self._group))

    def __getitem__(self, i):
        return self._books.pages(self._slot, self._group)[i]


class RequestRecord:
    """A live request as the books see it."""
    __slots__ = ("request_id", "slot", "pages", "_books")

    def __init__(self, request_id, slot: int, books: Books):
        self.request_id, self.slot, self._books = request_id, slot, books
        self.pages = [PageView(books, slot, g) for g in range(books.n_groups)]

    @property
    def length(self) -> int:                  # tokens whose keys/state are in the cache
        return self._books.length(self.slot)

    @property
    def reserved_to(self) -> int:             # positions [0, reserved_to) have pages (where still live)
        return self._books.reserved_to(self.slot)


class PoolView:
    """One group's page pool as the books see it."""

    def __init__(self, books: Books, group: int):
        self._books, self._group = books, group

    @property
    def n_pages(self) -> int:
        return self._books.pool_pages(self._group)

    @property
    def n_free(self) -> int:
        return self._books.free_pages()[self._group]

    @property
    def n_held(self) -> int:
        return self.n_pages - self.n_free

    def is_held(self, page: int) -> bool:
        return self._books.is_held(self._group, page)


class CacheGroup:
    def __init__(self, index: int, req: KVRequirement, owners: list, n_pages: int, page_size: int, device, dtype):
        self.index, self.req, self.owners = index, req, owners
        self.page_size = page_size
        self.n_pages = n_pages
        self.pool = None                      # a PoolView, set by the manager once the books exist
        shape = (n_pages, req.kv_heads, page_size, req.head_dim)
        # Zeroed once (the reference leaves its pools uninitialised, scratch.rs:546-573).  A key is always
        # written before any query can see it, but the tensor-core attention fetches whole pages, masked slots
        # included, and a masked probability of 0 times a stray NaN would still be NaN.
        self.k = {c: torch.zeros(shape, dtype=dtype, device=device) for c in owners}
        self.v = {c: torch.zeros(shape, dtype=dtype, device=device) for c in owners}

    def bytes_per_token(self) -> int:
        any_pool = next(iter(self.k.values()))
        return 2 * len(self.owners) * self.req.kv_heads * self.req.head_dim * any_pool.element_size()


@dataclass
class Snapshot:
    """What a request holds, copied to the host: its length, per group the first live page and the contents of
    the live pages of every layer call that owns a cache, and its fixed-size state."""
    length: int
    first_pages: list                          # per group
    k: dict = field(default_factory=dict)      # owner call -> host tensor [live pages, kv heads, page size, head size]
    v: dict = field(default_factory=dict)
    state: dict = field(default_factory=dict)  # call -> host tensor [*shape]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for d in (self.k, self.v, self.state) for t in d.values())


class CacheManager:
    def __init__(self, plans: list, *, max_tokens: int, page_size: int, max_requests: int, device, dtype,
                 max_seq_len: int | None = None, max_step_tokens: int | None = None):
        """max_seq_len: the most tokens a request may reach (default: what the pool holds); max_step_tokens:
        the most tokens one step brings for one request, which bounds the live pages of a windowed group and with
        them the width of its block table (default: no bound but max_seq_len)."""
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.device = device
        self.plans = plans
        n_pages = max(1, -(-int(max_tokens) // self.page_size))
        self.max_pages_per_request = -(-int(max_seq_len or max_tokens) // self.page_size)
        self.max_step_tokens = int(max_step_tokens) if max_step_tokens else None
        # ---- groups ----
        self.groups: list[CacheGroup] = []
        self.group_of_call: dict[int, int] = {}
        by_req: dict[KVRequirement, list] = {}
        for ci, plan in enumerate(plans):
            if plan.cache_from is not None:
                src = plans[plan.cache_from]
                if src.kv is None or src.cache_from is not None:
                    raise ValueError(f"call {ci} reads the cache of call {plan.cache_from}, which owns none")
                if plan.kv is not None and (plan.kv.kv_heads, plan.kv.head_dim) != (src.kv.kv_heads, src.kv.head_dim):
                    raise ValueError(f"call {ci} and call {plan.cache_from} disagree on the cache geometry")
                # pages are given back by the owner's window: a reader that looks further back than the owner
                # would ask for keys whose pages are gone
                if plan.kv is not None and src.kv.window > 0 and (plan.kv.window == 0 or plan.kv.window > src.kv.window):
                    raise ValueError(f"call {ci} reads the cache of call {plan.cache_from} with a window of "
                                     f"{plan.kv.window or 'all'} keys, but that cache keeps only {src.kv.window}")
                continue
            if plan.kv is not None:
                by_req.setdefault(plan.kv, []).append(ci)
        for gi, (req, owners) in enumerate(by_req.items()):
            self.groups.append(CacheGroup(gi, req, owners, n_pages, self.page_size, device, dtype))
            for c in owners:
                self.group_of_call[c] = gi
        for ci, plan in enumerate(plans):
            if plan.cache_from is not None:
                self.group_of_call[ci] = self.group_of_call[plan.cache_from]
        # ---- fixed-size state slots ----
        self.state: dict[int, torch.Tensor] = {}
        for ci, plan in enumerate(plans):
            if plan.state is not None:
                sd = dtype if plan.state.dtype == "engine" else getattr(torch, plan.state.dtype)
                self.state[ci] = torch.zeros((self.max_requests, *plan.state.shape), dtype=sd, device=device)
        self.books = Books([g.n_pages for g in self.groups], [g.req.window for g in self.groups], self.page_size,
                           self.max_requests, self.max_pages_per_request)
        # Columns of a block-table row: the most live pages a request holds in any group.  A group with a window W
        # keeps, while a step of k new tokens runs, the pages from position length - W + 1 to length + k.
        self.table_pages = 1
        for g in self.groups:
            live = self.max_pages_per_request
            if g.req.window > 0 and self.max_step_tokens:
                live = min(live, -(-(g.req.window + self.max_step_tokens) // self.page_size) + 2)
            self.table_pages = max(self.table_pages, live)
        for g in self.groups:
            g.pool = PoolView(self.books, g.index)
        self.requests: dict[object, RequestRecord] = {}

    # ---- sizes -------------------------------------------------------------
    @property
    def n_groups(self) -> int:
        return len(self.groups)

    def state_bytes_per_request(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self.state.values())

    def kv_bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)

    def free_pages(self) -> list:
        return self.books.free_pages()

    # ---- requests ----------------------------------------------------------
    def has_slot(self) -> bool:
        return self.books.has_slot()

    def admit(self, request_id) -> RequestRecord:
        if request_id in self.requests:
            raise PageError(f"request {request_id!r} is already live")
        slot = self.books.admit()
        for t in self.state.values():
            t[slot].zero_()                      # a fresh request starts from zero state
        rec = RequestRecord(request_id, slot, self.books)
        self.requests[request_id] = rec
        return rec

    def length(self, request_id) -> int:
        return self.requests[request_id].length

    def pages_needed(self, request_id, n_new: int) -> list:
        """Pages each group would have to take so that `n_new` more tokens fit."""
        return self.books.pages_needed(self.requests[request_id].slot, n_new)

    def can_reserve(self, needs: list) -> bool:
        """`needs` = list of (request_id, n_new) considered together."""
        return self.books.reserve_all([self.requests[rid].slot for rid, _ in needs], [k for _, k in needs],
                                      dry_run=True)

    def reserve(self, request_id, n_new: int) -> None:
        """Take the pages for positions [length, length + n_new) in every group, or none at all."""
        self.books.reserve_all([self.requests[request_id].slot], [n_new])

    def reserve_all(self, needs: list) -> None:
        """reserve() for several (request_id, n_new) at once: every request gets its pages, or none does."""
        self.books.reserve_all([self.requests[rid].slot for rid, _ in needs], [k for _, k in needs])

    def commit(self, request_id, n_new: int) -> None:
        """The step that wrote `n_new` tokens is launched: advance the length and give back the pages that
        no later query can see.  (Kernels of later steps run after this step's on the same stream, so a page
        that is reused is only overwritten after its last reader.)"""
        self.books.commit([self.requests[request_id].slot], [n_new])

    def commit_all(self, needs: list) -> None:
        self.books.commit([self.requests[rid].slot for rid, _ in needs], [k for _, k in needs])

    def release(self, request_id) -> None:
        rec = self.requests.pop(request_id)
        self.books.release(rec.slot)

    def release_all(self) -> None:
        for rid in list(self.requests):
            self.release(rid)

    # ---- snapshot and restore ------------------------------------------------
    def snapshot(self, request_id) -> Snapshot:
        """Copy what the request holds to the host (the copies are complete when this returns).  The request
        stays live; release it to give its pages to others.  The reference snapshots contiguous slots only and
        refuses paged ones (crates/forward/src/core/scratch.rs:1575-1581)."""
        rec = self.requests[request_id]
        snap = Snapshot(length=rec.length, first_pages=[self.books.first_live_page(rec.slot, g.index)
                                                        for g in self.groups])
        for g in self.groups:
            ids = [p for p in rec.pages[g.index] if p >= 0]
            # only pages that hold committed tokens (pages reserved ahead of the length hold nothing yet)
            ids = ids[:max(0, -(-rec.length // self.page_size) - snap.first_pages[g.index])]
            index = torch.tensor(ids, dtype=torch.long, device=self.device)
            for c in g.owners:
                snap.k[c] = g.k[c].index_select(0, index).cpu()
                snap.v[c] = g.v[c].index_select(0, index).cpu()
        for c, t in self.state.items():
            snap.state[c] = t[rec.slot].to("cpu", copy=True)
        return snap

    def restore(self, request_id, snap: Snapshot) -> RequestRecord:
        """Bring a snapshot back as a live request under `request_id`: a slot and fresh pages are taken (all or
        nothing, OutOfPages otherwise) and filled with the snapshot's contents; the request then continues at
        position snap.length as if it had never left."""
        if request_id in self.requests:
            raise PageError(f"request {request_id!r} is already live")
        if len(snap.first_pages) != self.n_groups:
            raise PageError("the snapshot was taken from a cache with other groups")
        slot = self.books.admit_at(snap.length, snap.first_pages)
        rec = RequestRecord(request_id, slot, self.books)
        self.requests[request_id] = rec
        for g in self.groups:
            ids = [p for p in rec.pages[g.index] if p >= 0]
            index = torch.tensor(ids, dtype=torch.long, device=self.device)
            for c in g.owners:
                if snap.k[c].shape[0] != len(ids):
                    self.release(request_id)
                    raise PageError("the snapshot does not fit this cache's page size")
                g.k[c].index_copy_(0, index, snap.k[c].to(self.device))
                g.v[c].index_copy_(0, index, snap.v[c].to(self.device))
        for c, t in self.state.items():
            t[slot].copy_(snap.state[c])
        return rec

    # ---- what a step needs ---------------------------------------------------
    def table_row(self, request_id, group: int) -> list:
        return self.requests[request_id].pages[group]

    def view(self, call: int, tables: list, table_bases: list | None = None) -> LayerCacheView:
        """The cache as call `call` of the run order sees it; `tables[g]` is the device block table of
        group g for the sequences of this step and `table_bases[g]` the logical page its rows start at."""
        plan = self.plans[call]
        state = self.state.get(call)
        gi = self.group_of_call.get(call)
        if gi is None:
            return LayerCacheView(None, None, None, None, self.page_size, False, -1, state)
        owner = plan.cache_from if plan.cache_from is not None else call
        g = self.groups[gi]
        return LayerCacheView(g.k[owner], g.v[owner], tables[gi], table_bases[gi] if table_bases else None,
                              self.page_size, plan.cache_from is None, gi, state)

    def first_live_page(self, request_id, group: int) -> int:
        """The logical page index that the request's block-table row starts at in `group`."""
        return self.books.first_live_page(self.requests[request_id].slot, group)

    # ---- invariants (used by tests) ------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, held twice or free while in a table; no slot held twice; the ids and the books agree."""
        self.books.check_invariants()
        slots = [r.slot for r in self.requests.values()]
        if len(set(slots)) != len(slots):
            raise PageError("a request slot is held twice")
