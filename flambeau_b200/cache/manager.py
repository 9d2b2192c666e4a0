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

The manager, not the caller, owns each request's length.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..parts.base import KVRequirement, StateRequirement
from .pages import OutOfPages, PageError, PageList, PagePool


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
    block_table: Optional[torch.Tensor]       # device int32 [sequences of the step, pages per request]
    page_size: int
    writable: bool
    group: int
    state: Optional[torch.Tensor] = None      # [slots, *shape] for mixers with fixed-size state


@dataclass
class RequestRecord:
    request_id: object
    slot: int
    length: int = 0                           # tokens whose keys/state are in the cache
    pages: list = field(default_factory=list)         # per group: list of physical page ids, -1 = given back
    reserved_to: int = 0                      # positions [0, reserved_to) have pages (where still live)


class CacheGroup:
    def __init__(self, index: int, req: KVRequirement, owners: list, n_pages: int, page_size: int, device, dtype):
        self.index, self.req, self.owners = index, req, owners
        self.page_size = page_size
        self.pool = PagePool(n_pages)
        shape = (n_pages, req.kv_heads, page_size, req.head_dim)
        # Zeroed once (the reference leaves its pools uninitialised, scratch.rs:546-573).  A key is always
        # written before any query can see it, but the tensor-core attention fetches whole pages, masked slots
        # included, and a masked probability of 0 times a stray NaN would still be NaN.
        self.k = {c: torch.zeros(shape, dtype=dtype, device=device) for c in owners}
        self.v = {c: torch.zeros(shape, dtype=dtype, device=device) for c in owners}

    def bytes_per_token(self) -> int:
        any_pool = next(iter(self.k.values()))
        return 2 * len(self.owners) * self.req.kv_heads * self.req.head_dim * any_pool.element_size()


class CacheManager:
    def __init__(self, plans: list, *, max_tokens: int, page_size: int, max_requests: int, device, dtype,
                 max_seq_len: int | None = None):
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.device = device
        self.plans = plans
        n_pages = max(1, -(-int(max_tokens) // self.page_size))
        self.max_pages_per_request = -(-int(max_seq_len or max_tokens) // self.page_size)
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
        self._free_slots = list(range(self.max_requests - 1, -1, -1))
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
        return [g.pool.n_free for g in self.groups]

    # ---- requests ----------------------------------------------------------
    def has_slot(self) -> bool:
        return bool(self._free_slots)

    def admit(self, request_id) -> RequestRecord:
        if request_id in self.requests:
            raise PageError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise PageError(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        for t in self.state.values():
            t[slot].zero_()                      # a fresh request starts from zero state
        rec = RequestRecord(request_id, slot, pages=[PageList() for _ in self.groups])
        self.requests[request_id] = rec
        return rec

    def length(self, request_id) -> int:
        return self.requests[request_id].length

    def pages_needed(self, request_id, n_new: int) -> list:
        """Pages each group would have to take so that `n_new` more tokens fit."""
        rec = self.requests[request_id]
        want = -(-(rec.length + n_new) // self.page_size)
        return [max(0, want - len(rec.pages[g.index])) for g in self.groups]

    def can_reserve(self, needs: list) -> bool:
        """`needs` = list of (request_id, n_new) considered together."""
        total = [0] * len(self.groups)
        for rid, n_new in needs:
            for gi, k in enumerate(self.pages_needed(rid, n_new)):
                total[gi] += k
        return all(total[gi] <= g.pool.n_free for gi, g in enumerate(self.groups))

    def reserve(self, request_id, n_new: int) -> None:
        """Take the pages for positions [length, length + n_new) in every group, or none at all."""
        rec = self.requests[request_id]
        end = rec.length + n_new
        if end > self.max_pages_per_request * self.page_size:
            raise PageError(f"request {request_id!r} would reach {end} tokens; the cache holds at most "
                            f"{self.max_pages_per_request * self.page_size} per request")
        needs = self.pages_needed(request_id, n_new)
        for gi, g in enumerate(self.groups):
            if needs[gi] > g.pool.n_free:
                raise OutOfPages(needs[gi], g.pool.n_free, g.pool.n_pages)
        for gi, g in enumerate(self.groups):
            rec.pages[gi].extend(g.pool.take(needs[gi]))
        rec.reserved_to = max(rec.reserved_to, end)

    def reserve_all(self, needs: list) -> None:
        """reserve() for several (request_id, n_new) at once: every request gets its pages, or none does."""
        page, limit = self.page_size, self.max_pages_per_request * self.page_size
        want = []
        total = [0] * len(self.groups)
        for rid, n_new in needs:
            rec = self.requests[rid]
            end = rec.length + n_new
            if end > limit:
                raise PageError(f"request {rid!r} would reach {end} tokens; the cache holds at most {limit} per request")
            pages_to = -(-end // page)
            row = [max(0, pages_to - len(rec.pages[gi])) for gi in range(len(self.groups))]
            for gi, k in enumerate(row):
                total[gi] += k
            want.append((rec, end, row))
        for gi, g in enumerate(self.groups):
            if total[gi] > g.pool.n_free:
                raise OutOfPages(total[gi], g.pool.n_free, g.pool.n_pages)
        for rec, end, row in want:
            for gi, k in enumerate(row):
                if k:
                    rec.pages[gi].extend(self.groups[gi].pool.take(k))
            rec.reserved_to = max(rec.reserved_to, end)

    def commit(self, request_id, n_new: int) -> None:
        """The step that wrote `n_new` tokens is launched: advance the length and give back the pages that
        no later query can see.  (Kernels of later steps run after this step's on the same stream, so a page
        that is reused is only overwritten after its last reader.)"""
        rec = self.requests[request_id]
        rec.length += n_new
        if rec.length > rec.reserved_to:
            raise PageError(f"request {request_id!r}: {rec.length} tokens committed, {rec.reserved_to} reserved")
        for gi, g in enumerate(self.groups):
            w = g.req.window
            if w <= 0:
                continue
            first_live = rec.length - w + 1           # lowest position a future query can see
            dead_pages = max(0, first_live) // self.page_size
            back = rec.pages[gi].give_back_prefix(dead_pages)
            if back:
                g.pool.give_back(back)

    def release(self, request_id) -> None:
        rec = self.requests.pop(request_id)
        for gi, g in enumerate(self.groups):
            g.pool.give_back(rec.pages[gi].live())
            rec.pages[gi] = PageList()
        self._free_slots.append(rec.slot)

    def release_all(self) -> None:
        for rid in list(self.requests):
            self.release(rid)

    # ---- what a step needs ---------------------------------------------------
    def table_row(self, request_id, group: int) -> list:
        return self.requests[request_id].pages[group]

    def view(self, call: int, tables: list) -> LayerCacheView:
        """The cache as call `call` of the run order sees it; `tables[g]` is the device block table of
        group g for the sequences of this step."""
        plan = self.plans[call]
        state = self.state.get(call)
        gi = self.group_of_call.get(call)
        if gi is None:
            return LayerCacheView(None, None, None, self.page_size, False, -1, state)
        owner = plan.cache_from if plan.cache_from is not None else call
        g = self.groups[gi]
        return LayerCacheView(g.k[owner], g.v[owner], tables[gi], self.page_size,
                              plan.cache_from is None, gi, state)

    # ---- invariants (used by tests) ------------------------------------------
    def check_invariants(self) -> None:
        for gi, g in enumerate(self.groups):
            seen = set()
            for rec in self.requests.values():
                for p in rec.pages[gi]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise PageError(f"group {gi}: page {p} is held twice")
                    if not g.pool.is_held(p):
                        raise PageError(f"group {gi}: page {p} is in a table but free in the pool")
                    seen.add(p)
            if len(seen) != g.pool.n_held:
                raise PageError(f"group {gi}: {g.pool.n_held} pages held in the pool, {len(seen)} in tables (lost pages)")
        slots = [r.slot for r in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise PageError("a request slot is held twice")
