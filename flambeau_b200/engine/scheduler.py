"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.

One loop owns the engine; every iteration builds one step.  Every running
request that has its prompt in the cache contributes one row (its last sampled
token); what is left of the step's token budget is filled with portions of the
prompts that are still being fed, in arrival order.  The reference reaches the
same mix with a thread per request, a pending queue and a leader that drains
it (crates/server/src/routes.rs:577-733, 753-821;
crates/server/src/routes/decode_loop.rs:365-520).

When pages run out the reference fails the forward call
(crates/forward/src/core/composites/standard_attn.rs:449-458).  Here no step
fails for lack of pages:
  * beside running requests, a request is admitted only if its whole prompt
    (what a window keeps of it) and its first token fit into the pages that
    are free after the running requests' prompts have taken theirs, and its
    first portion fits with a page of headroom for every running request;
    with nothing running, if its first portion fits;
  * a prompt portion is shortened to the pages that are free, or waits;
  * if the decoding requests cannot all get the page their next token needs,
    the youngest running request is preempted: its pages are given back and it
    returns to the front of the queue with prompt := prompt + generated so far,
    to be fed again later (its draws continue where they stopped);
  * if nothing can be scheduled although requests are running (all of them
    in the middle of their prompts, no page free), the youngest is preempted
    in the same way;
  * a request that cannot fit even alone is finished with reason 'capacity';
    one that reaches the most tokens a request may hold (the engine's
    max_seq_len; --ctx-cap) ends with reason 'length', as at max_tokens.

Running ahead.  While every running request is decoding and none is about to reach its token limit, the next
step is known but for the token ids, and those are on the device: the scheduler queues it (token ids fed from the
sampler's output buffer) before it reads the tokens of the step that is running, so the device never waits for
the host.  A request that turns out to have stopped in the meantime has one row too many in the step already
queued; that row's token is dropped.  What is generated does not change: a request's logits do not depend on the
other rows of its step, and its draws are numbered.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..sampling.params import SamplingParams
from .batch import Entry


@dataclass
class Request:
    request_id: object
    prompt: list
    params: SamplingParams = field(default_factory=SamplingParams)
    generated: list = field(default_factory=list)
    fed: int = 0                       # tokens of prompt+generated whose keys are in the cache
    arrival: int = 0
    finish_reason: Optional[str] = None
    preemptions: int = 0

    @property
    def tokens(self) -> list:
        return self.prompt + self.generated

    def span(self, a: int, b: int) -> list:
        """tokens[a:b] of prompt + generated without building the whole list."""
        p = len(self.prompt)
        if b <= p:
            return self.prompt[a:b]
        if a >= p:
            return self.generated[a - p:b - p]
        return self.prompt[a:] + self.generated[:b - p]

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.generated) - self.fed

    @property
    def decoding(self) -> bool:
        return self.remaining == 1 and bool(self.generated)


@dataclass
class PlannedStep:
    entries: list                      # engine.batch.Entry
    sampled: list                      # requests whose last row's logits are sampled, in the order of the wanted rows
    preempted: list
    admitted: list


class Scheduler:
    def __init__(self, executor, *, token_budget: int = 2048, prefill_chunk: int = 2048, max_running: int = 4,
                 run_ahead: bool = True):
        """`executor` has .cache (a CacheManager), .run(entries, sampled_requests) -> list of token ids, and
        .finish(request_id); for running ahead also .launch(entries, sampled, feed, pending) -> handle,
        .collect(handle) -> list of token ids and .can_run_ahead(sampled)."""
        if token_budget < 1 or prefill_chunk < 1 or max_running < 1:
            raise ValueError("token_budget, prefill_chunk and max_running must be positive")
        self.executor = executor
        self.cache = executor.cache
        # never more running requests than the cache has slots for per-request state
        max_running = min(max_running, getattr(self.cache, "max_requests", max_running))
        self.token_budget, self.prefill_chunk, self.max_running = token_budget, prefill_chunk, max_running
        self.waiting: deque = deque()
        self.running: list = []
        self.finished: list = []
        self._arrivals = 0
        self.steps = 0
        # the most tokens one request may hold (prompt and generated together); None: no limit but the pool
        self.max_request_tokens = getattr(executor, "max_request_tokens", None)
        self._two_phase = all(hasattr(executor, m) for m in ("launch", "collect", "can_run_ahead"))
        self.run_ahead = run_ahead and self._two_phase      # may be switched while running
        self._ahead = None                 # (PlannedStep, handle) of a step that is queued but not collected
        self.steps_ahead = 0               # steps that were queued ahead

    # ---- requests ----------------------------------------------------------------
    def add(self, request_id, prompt, params: SamplingParams | None = None) -> Request:
        if not prompt:
            raise ValueError("a request needs at least one prompt token")   # decode_loop.rs:532-534
        r = Request(request_id, list(prompt), params or SamplingParams(), arrival=self._arrivals)
        self._arrivals += 1
        if r.params.max_tokens == 0:
            r.finish_reason = "length"
            self.finished.append(r)
        elif self.max_request_tokens is not None and len(r.prompt) > self.max_request_tokens:
            r.finish_reason = "capacity"                   # the prompt alone is longer than a request may be
            self.finished.append(r)
        else:
            self.waiting.append(r)
        return r

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running and self._ahead is None

    # ---- planning ----------------------------------------------------------------
    def _pages_free(self) -> list:
        return list(self.cache.free_pages())

    def _fits(self, free: list, need: list) -> bool:
        return all(n <= f for n, f in zip(need, free))

    def _preempt(self, r: Request, plan: PlannedStep) -> None:
        self.cache.release(r.request_id)
        self.running.remove(r)
        r.fed = 0
        r.preemptions += 1
        self.waiting.appendleft(r)
        plan.preempted.append(r)

    def _finish(self, r: Request, reason: str) -> None:
        r.finish_reason = reason
        if r in self.running:
            self.running.remove(r)
        if r.request_id in self.cache.requests:
            self.executor.finish(r.request_id)
        self.finished.append(r)

    def plan(self) -> PlannedStep:
        """Decide the next step.  Takes no pages itself (the engine's step reserves them), but preempts and
        admits as needed, so that the planned entries are sure to fit."""
        plan = PlannedStep([], [], [], [])
        while True:
            self._plan_once(plan)
            if plan.entries or not self.running:
                return plan
            # every running request is in the middle of its prompt and no page is free: the youngest gives way
            victim = max(self.running, key=lambda r: r.arrival)
            if len(self.running) == 1:
                self._finish(victim, "capacity")
            else:
                self._preempt(victim, plan)

    def _pages_for(self, tokens: int, group: int) -> int:
        """Pages that `tokens` tokens of one request hold in a group at most (a window keeps the last W tokens,
        plus the portion that is being written and the page the window starts in)."""
        window = self.cache.groups[group].req.window
        page = self.cache.page_size
        if window:
            tokens = min(tokens, window + self.prefill_chunk + page)
        return -(-tokens // page)

    def _plan_once(self, plan: PlannedStep) -> None:
        budget = self.token_budget
        cache = self.cache
        page = cache.page_size

        # 1. decoding requests, oldest first; make room by preempting the youngest running request
        decoders = sorted((r for r in self.running if r.decoding), key=lambda r: r.arrival)
        while True:
            need = [0] * cache.n_groups
            for r in decoders[:budget]:
                for gi, k in enumerate(cache.pages_needed(r.request_id, 1)):
                    need[gi] += k
            if self._fits(self._pages_free(), need):
                break
            victim = max(self.running, key=lambda r: r.arrival)
            if len(self.running) == 1:
                self._finish(victim, "capacity")          # it cannot fit even alone
            else:
                self._preempt(victim, plan)
            decoders = [r for r in decoders if r in self.running]
        free = self._pages_free()
        for r in decoders[:budget]:
            for gi, k in enumerate(cache.pages_needed(r.request_id, 1)):
                free[gi] -= k
            plan.entries.append(Entry(r.request_id, [r.generated[-1]], [0]))
            plan.sampled.append(r)
            budget -= 1

        # 2. portions of prompts that are being fed, in arrival order; 3. admissions, in queue order
        def portion(r: Request, headroom: int) -> int:
            """Longest portion of r that budget, chunk size and free pages (less headroom) allow."""
            k = min(r.remaining, self.prefill_chunk, budget)
            held = cache.length(r.request_id) if r.request_id in cache.requests else 0
            for gi in range(cache.n_groups):
                have = len(cache.requests[r.request_id].pages[gi]) if r.request_id in cache.requests else 0
                room = (have + max(0, free[gi] - headroom)) * page - held
                k = min(k, room)
            return max(k, 0)

        def take(r: Request, k: int) -> None:
            nonlocal budget
            toks = r.span(r.fed, r.fed + k)
            last = r.fed + k == len(r.prompt) + len(r.generated)
            if r.request_id in cache.requests:
                need = cache.pages_needed(r.request_id, k)
            else:
                need = [-(-k // page)] * cache.n_groups
            for gi, n in enumerate(need):
                free[gi] -= n
            plan.entries.append(Entry(r.request_id, toks, [k - 1] if last else []))
            if last:
                plan.sampled.append(r)
            budget -= k

        for r in sorted((r for r in self.running if not r.decoding), key=lambda r: r.arrival):
            if budget <= 0:
                break
            k = portion(r, 0)
            if k > 0:
                take(r, k)
        # pages that the running requests' prompts will still take (this step's portions among them)
        owed = [0] * cache.n_groups
        for r in self.running:
            for gi in range(cache.n_groups):
                have = len(cache.requests[r.request_id].pages[gi]) if r.request_id in cache.requests else 0
                owed[gi] += max(0, self._pages_for(len(r.prompt) + len(r.generated) + 1, gi) - have)
        free_now = self._pages_free()
        while self.waiting and budget > 0 and len(self.running) < self.max_running and cache.has_slot():
            r = self.waiting[0]
            k = portion(r, headroom=len(self.running))
            whole = [self._pages_for(len(r.prompt) + len(r.generated) + 1, gi) for gi in range(cache.n_groups)]
            if self.running and any(whole[gi] + owed[gi] > free_now[gi]
                                    for gi in range(cache.n_groups)):
                k = 0                                     # it would starve the prompts that are being fed
            if k <= 0:
                if not self.running and not plan.entries:
                    # alone, with every page free, and still no room for one token
                    self.waiting.popleft()
                    self._finish(r, "capacity")
                    continue
                break
            self.waiting.popleft()
            self.running.append(r)
            plan.admitted.append(r)
            take(r, k)
            for gi in range(cache.n_groups):
                owed[gi] += whole[gi]

    # ---- running -----------------------------------------------------------------
    def step(self) -> list:
        """Plan and run one step (or collect the one that was queued ahead); returns [(request, token)] for the
        tokens sampled in it."""
        tokens = None
        if self._ahead is not None:
            plan, handle = self._ahead
            self._ahead = None
        else:
            plan = self.plan()
            if not plan.entries:
                if self.running or self.waiting:
                    # nothing could be scheduled although work is left: the head of the queue can never fit
                    if self.waiting and not self.running:
                        self._finish(self.waiting.popleft(), "capacity")
                        return []
                    raise RuntimeError("scheduler: running requests but nothing to run")
                return []
            if self._two_phase:
                handle = self.executor.launch(plan.entries, plan.sampled)
            else:
                handle = None
                tokens = self.executor.run(plan.entries, plan.sampled)
        self.steps += 1
        if tokens is None:
            if self.run_ahead:
                self._queue_ahead(plan, handle)
            tokens = self.executor.collect(handle) if handle is not None else []
        by_id = {r.request_id: r for r in self.running}
        for e in plan.entries:
            if e.request_id in by_id:                      # (a request that stopped has left meanwhile)
                by_id[e.request_id].fed += len(e.tokens)
        out = []
        for r, tok in zip(plan.sampled, tokens):
            if r.finish_reason is not None:
                continue                                   # it stopped in the step before: a row too many
            r.generated.append(int(tok))
            out.append((r, int(tok)))
            if not r.params.ignore_eos and int(tok) in r.params.stop_token_ids:
                self._finish(r, "stop")
            elif len(r.generated) >= r.params.max_tokens or self._at_limit(r, 0):
                self._finish(r, "length")
        return out

    def _at_limit(self, r: Request, more: int) -> bool:
        """With `more` further tokens the request would hold as many tokens as one request may."""
        return self.max_request_tokens is not None and \
            len(r.prompt) + len(r.generated) + more >= self.max_request_tokens

    def _queue_ahead(self, plan: PlannedStep, handle) -> None:
        """Queue the step after `plan` (whose tokens are not known yet) if it is sure to be one decoded token for
        every running request."""
        if handle is None or self.waiting or not self.running:
            return
        sampled = plan.sampled
        if len(sampled) != len(self.running) or len(sampled) > self.token_budget:
            return
        live = set(id(r) for r in self.running)
        for r in sampled:
            # running, its whole prompt fed by `plan`, and not at its limit with the token that is on its way
            if id(r) not in live or r.finish_reason is not None or len(r.generated) + 2 > r.params.max_tokens \
                    or self._at_limit(r, 1):
                return
        fed_by_plan = {e.request_id: len(e.tokens) for e in plan.entries}
        for r in sampled:
            if r.remaining - fed_by_plan.get(r.request_id, 0) != 0:
                return
        if not self.executor.can_run_ahead(sampled):
            return
        need = [0] * self.cache.n_groups
        for r in sampled:
            for gi, k in enumerate(self.cache.pages_needed(r.request_id, 1)):
                need[gi] += k
        if not self._fits(self._pages_free(), need):
            return                                         # the planner will make room, knowing the tokens
        entries = [Entry(r.request_id, [0], [0]) for r in sampled]          # the ids come from the device
        nxt = PlannedStep(entries, list(sampled), [], [])
        self._ahead = (nxt, self.executor.launch(entries, sampled, feed=handle, pending=1))
        self.steps_ahead += 1

    def run(self) -> list:
        """Run until every request has finished; returns them in arrival order."""
        while not self.idle:
            self.step()
        return sorted(self.finished, key=lambda r: r.arrival)
