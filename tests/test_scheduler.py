"""The scheduler's decisions on the CPU, with an executor that keeps the cache books but computes nothing."""
import pytest
import torch

from flambeau_b200.cache.manager import CacheManager, CallPlan
from flambeau_b200.engine.scheduler import Scheduler
from flambeau_b200.parts.base import KVRequirement
from flambeau_b200.sampling.params import SamplingParams


class BookkeepingExecutor:
    """Does what Engine.step does to the cache (admit, reserve all-or-nothing, commit) and returns token ids
    that encode who was sampled when, so that tests can follow the order of events."""

    def __init__(self, tokens=256, window=0, max_requests=4, page_size=16):
        self.cache = CacheManager([CallPlan(kv=KVRequirement(1, 8, window))], max_tokens=tokens, page_size=page_size,
                                  max_requests=max_requests, device="cpu", dtype=torch.float32, max_seq_len=4096)
        self.log = []

    def run(self, entries, sampled):
        for e in entries:
            if e.request_id not in self.cache.requests:
                self.cache.admit(e.request_id)
        assert self.cache.can_reserve([(e.request_id, len(e.tokens)) for e in entries]), "planned step does not fit"
        for e in entries:
            self.cache.reserve(e.request_id, len(e.tokens))
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.cache.check_invariants()
        self.log.append([(e.request_id, len(e.tokens), list(e.want)) for e in entries])
        want_ids = [e.request_id for e in entries if e.want]
        assert want_ids == [r.request_id for r in sampled]
        return [100 + len(r.generated) for r in sampled]

    def finish(self, request_id):
        self.cache.release(request_id)


def test_prompt_is_cut_under_the_budget_and_decodes_come_first():
    ex = BookkeepingExecutor()
    s = Scheduler(ex, token_budget=16, prefill_chunk=10, max_running=4)
    s.add("a", list(range(25)), SamplingParams(max_tokens=3))
    s.step()
    assert ex.log[-1] == [("a", 10, [])]                        # chunk limit
    s.add("b", list(range(30)), SamplingParams(max_tokens=2))
    s.step()
    assert ex.log[-1] == [("a", 10, []), ("b", 6, [])]          # budget 16 = 10 + 6, arrival order
    s.step()
    assert ex.log[-1] == [("a", 5, [4]), ("b", 10, [])]         # a's prompt ends: its last row is wanted
    s.step()
    assert ex.log[-1] == [("a", 1, [0]), ("b", 10, [])]         # a decodes beside b's portion
    s.step()
    assert ex.log[-1] == [("a", 1, [0]), ("b", 4, [3])]
    done = s.run()
    assert [r.request_id for r in done] == ["a", "b"]
    assert done[0].generated == [100, 101, 102] and done[0].finish_reason == "length"
    assert done[1].generated == [100, 101]
    assert not ex.cache.requests and ex.cache.free_pages() == [16]


def test_positions_first_generated_token_is_fed_at_prompt_length():
    ex = BookkeepingExecutor()
    s = Scheduler(ex, token_budget=64, prefill_chunk=64)
    r = s.add("a", [1, 2, 3, 4, 5], SamplingParams(max_tokens=4))
    s.step()
    assert ex.cache.length("a") == 5 and r.generated == [100]
    s.step()
    assert ex.cache.length("a") == 6                            # the token sampled from position 4 sits at 5


def test_stop_token_and_max_tokens_zero():
    ex = BookkeepingExecutor()
    s = Scheduler(ex)
    a = s.add("a", [1, 2], SamplingParams(max_tokens=10, stop_token_ids=(101,)))
    b = s.add("b", [1, 2], SamplingParams(max_tokens=10, stop_token_ids=(101,), ignore_eos=True))
    c = s.add("c", [1], SamplingParams(max_tokens=0))
    s.run()
    assert a.generated == [100, 101] and a.finish_reason == "stop"
    assert len(b.generated) == 10 and b.finish_reason == "length"
    assert c.generated == [] and c.finish_reason == "length"
    with pytest.raises(ValueError):
        s.add("d", [])


def test_admission_waits_for_a_slot_and_for_pages():
    ex = BookkeepingExecutor(tokens=64, max_requests=2)        # 4 pages, 2 slots
    s = Scheduler(ex, token_budget=64, prefill_chunk=64, max_running=4)
    for name in "abc":
        s.add(name, list(range(20)), SamplingParams(max_tokens=2))
    s.step()
    assert [e[0] for e in ex.log[-1]] == ["a", "b"]             # two slots; c waits
    assert [r.request_id for r in s.waiting] == ["c"]
    s.run()
    assert sorted(r.request_id for r in s.finished) == ["a", "b", "c"]
    assert all(len(r.generated) == 2 for r in s.finished)
    assert ex.cache.free_pages() == [4]


def test_out_of_pages_preempts_the_youngest_and_resumes_it():
    ex = BookkeepingExecutor(tokens=64, max_requests=4)         # 4 pages of 16
    s = Scheduler(ex, token_budget=64, prefill_chunk=64, max_running=4)
    a = s.add("a", list(range(30)), SamplingParams(max_tokens=20))   # will need 4 pages alone (50 tokens)
    b = s.add("b", list(range(14)), SamplingParams(max_tokens=40))
    preempted = []
    while not s.idle:
        before = len(s.finished)
        plan_preempted = len([r for r in (a, b) if r.preemptions])
        s.step()
        ex.cache.check_invariants()
    assert b.preemptions >= 1 and a.preemptions == 0, "the younger request gives way"
    assert a.finish_reason == "length" and len(a.generated) == 20
    assert b.finish_reason == "length" and len(b.generated) == 40
    # a preempted request is fed again from position 0 with prompt + generated so far
    refeeds = [e for step in ex.log for e in step if e[0] == "b" and e[1] > 1]
    assert len(refeeds) >= 2 and refeeds[-1][1] > 14
    assert ex.cache.free_pages() == [4] and not ex.cache.requests


def test_a_request_that_cannot_fit_alone_ends_with_capacity():
    ex = BookkeepingExecutor(tokens=32)                         # 2 pages
    s = Scheduler(ex, token_budget=64, prefill_chunk=64)
    a = s.add("a", list(range(20)), SamplingParams(max_tokens=30))
    b = s.add("b", list(range(5)), SamplingParams(max_tokens=3))
    s.run()
    assert a.finish_reason == "capacity" and 0 < len(a.generated) < 30
    assert b.finish_reason == "length" and len(b.generated) == 3
    assert ex.cache.free_pages() == [2]


def test_window_lets_a_long_request_run_in_a_small_pool():
    ex = BookkeepingExecutor(tokens=64, window=16)             # 4 pages, but only ~2 stay live per request
    s = Scheduler(ex, token_budget=8, prefill_chunk=8)
    a = s.add("a", list(range(40)), SamplingParams(max_tokens=100))
    s.run()
    assert a.finish_reason == "length" and len(a.generated) == 100 and a.preemptions == 0
    assert ex.cache.free_pages() == [4]


def test_random_load_never_breaks_the_books():
    import random
    rng = random.Random(3)
    ex = BookkeepingExecutor(tokens=160, max_requests=4)
    s = Scheduler(ex, token_budget=24, prefill_chunk=16, max_running=4)
    reqs = [s.add(i, list(range(rng.randint(1, 60))), SamplingParams(max_tokens=rng.randint(1, 40)))
            for i in range(12)]
    steps = 0
    while not s.idle:
        s.step()
        steps += 1
        assert steps < 5000
        assert sum(n for _, n, _ in ex.log[-1]) <= 24 if ex.log else True
    assert all(r.finish_reason == "length" and len(r.generated) == r.params.max_tokens for r in reqs)
    assert ex.cache.free_pages() == [10] and not ex.cache.requests


def test_a_request_ends_at_the_most_tokens_a_request_may_hold():
    for ahead in (False, True):
        ex = TwoPhaseExecutor(tokens=256, max_requests=4)
        ex.max_request_tokens = 20
        s = Scheduler(ex, token_budget=32, prefill_chunk=8, max_running=4, run_ahead=ahead)
        a = s.add("a", list(range(12)), SamplingParams(max_tokens=50))     # 12 + 8 = 20: stops there
        b = s.add("b", list(range(5)), SamplingParams(max_tokens=6))       # its own limit comes first
        c = s.add("c", list(range(20)), SamplingParams(max_tokens=6))      # the prompt fills it: one token
        d = s.add("d", list(range(21)), SamplingParams(max_tokens=6))      # longer than a request may be
        s.run()
        assert (len(a.generated), a.finish_reason) == (8, "length")
        assert (len(b.generated), b.finish_reason) == (6, "length")
        assert (len(c.generated), c.finish_reason) == (1, "length")
        assert (len(d.generated), d.finish_reason) == (0, "capacity")
        assert not ex.cache.requests and ex.in_flight == 0


def test_prompts_that_do_not_fit_together_are_not_fed_side_by_side():
    """Four prompts of 68 to 90 tokens and a pool of 256: fed side by side they would fill the pool with all four
    in mid-prompt and nothing could run.  The fourth waits until pages are free."""
    ex = BookkeepingExecutor(tokens=256, max_requests=8)
    s = Scheduler(ex, token_budget=96, prefill_chunk=16, max_running=8)
    reqs = [s.add(i, list(range(n)), SamplingParams(max_tokens=m))
            for i, (n, m) in enumerate([(79, 18), (90, 43), (84, 26), (68, 15)])]
    s.step()
    assert [e[0] for e in ex.log[-1]] == [0, 1]               # 5 + 6 pages of 16 are spoken for; 2 would need 6 more
    s.run()
    assert all(r.finish_reason == "length" and len(r.generated) == r.params.max_tokens for r in reqs)
    assert ex.cache.free_pages() == [16] and not ex.cache.requests


def test_running_requests_stuck_in_mid_prompt_make_the_youngest_give_way():
    """The state that admission now avoids, built by hand: two running requests in mid-prompt hold every page."""
    ex = BookkeepingExecutor(tokens=64, max_requests=4)        # 4 pages of 16
    s = Scheduler(ex, token_budget=64, prefill_chunk=32, max_running=4)
    a = s.add("a", list(range(60)), SamplingParams(max_tokens=2))
    b = s.add("b", list(range(60)), SamplingParams(max_tokens=2))
    for r in (a, b):                                           # as if both had been admitted and fed 32 tokens
        s.waiting.remove(r)
        s.running.append(r)
        ex.cache.admit(r.request_id)
        ex.cache.reserve(r.request_id, 32)
        ex.cache.commit(r.request_id, 32)
        r.fed = 32
    assert ex.cache.free_pages() == [0]
    s.step()
    assert b.preemptions == 1 and [e[0] for e in ex.log[-1]] == ["a"]
    s.run()
    assert a.finish_reason == b.finish_reason == "length" and len(b.generated) == 2
    assert ex.cache.free_pages() == [4]


@pytest.mark.parametrize("block", range(6))
def test_random_loads_pools_and_windows_always_end(block):
    """Random loads on random pools (down to three pages), windows, slots, budgets and portion sizes, with and
    without running ahead: every run ends, the books balance, every request gets its tokens, and 'capacity' is
    given only to a request that would not fit alone."""
    import random
    for seed in range(block * 50, block * 50 + 50):
        rng = random.Random(seed)
        n = rng.randint(1, 12)
        page = rng.choice([8, 16])
        pool = page * rng.randint(3, 24)
        window = rng.choice([0, 0, 0, 24, 40])
        slots = rng.choice([1, 2, 4, 8])
        lengths = [rng.randint(1, 120) for _ in range(n)]
        limits = [rng.randint(1, 60) for _ in range(n)]
        ex = TwoPhaseExecutor(tokens=pool, max_requests=slots, window=window, page_size=page)
        s = Scheduler(ex, token_budget=rng.choice([8, 24, 96]), prefill_chunk=rng.choice([4, 16, 33, 64]),
                      max_running=rng.choice([slots, 4]), run_ahead=rng.random() < 0.5)
        reqs = [s.add(i, list(range(l)), SamplingParams(max_tokens=m)) for i, (l, m) in enumerate(zip(lengths, limits))]
        steps = 0
        while not s.idle:
            s.step()
            steps += 1
            assert steps < 20000, f"seed {seed}: no end"
        ex.cache.check_invariants()
        assert not ex.cache.requests and ex.in_flight == 0, f"seed {seed}"
        for r in reqs:
            if r.finish_reason == "capacity":
                total = len(r.prompt) + r.params.max_tokens
                assert not (total <= pool or (window and pool >= window + 3 * page)), \
                    f"seed {seed}: request {r.request_id} fits alone but ended with 'capacity'"
            else:
                assert r.finish_reason == "length" and len(r.generated) == r.params.max_tokens, f"seed {seed}"


class TwoPhaseExecutor(BookkeepingExecutor):
    """The same books with the launch / collect interface: a step is queued with `launch`, its tokens are read
    later with `collect`; `pending` tokens of a request are on their way when its row is queued."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.in_flight = 0
        self.most_in_flight = 0
        self.fed_from_device = 0

    def launch(self, entries, sampled, feed=None, pending=0):
        if feed is not None:
            assert all(len(e.tokens) == 1 for e in entries) and len(feed) == len(entries)
            self.fed_from_device += 1
        if True:
            for e in entries:
                if e.request_id not in self.cache.requests:
                    self.cache.admit(e.request_id)
            assert self.cache.can_reserve([(e.request_id, len(e.tokens)) for e in entries])
            for e in entries:
                self.cache.reserve(e.request_id, len(e.tokens))
                self.cache.commit(e.request_id, len(e.tokens))
            self.log.append([(e.request_id, len(e.tokens), list(e.want)) for e in entries])
        if not sampled:
            return None
        self.in_flight += 1
        self.most_in_flight = max(self.most_in_flight, self.in_flight)
        return [100 + len(r.generated) + pending for r in sampled]

    def collect(self, handle):
        self.in_flight -= 1
        return handle

    def can_run_ahead(self, sampled):
        return all(not r.params.has_penalties for r in sampled)


def run_both(add_requests, **kw):
    results = []
    for ahead in (False, True):
        ex = TwoPhaseExecutor()
        s = Scheduler(ex, run_ahead=ahead, **kw)
        reqs = add_requests(s)
        s.run()
        ex.cache.check_invariants()
        assert not ex.cache.requests and ex.in_flight == 0
        results.append((ex, s, [(r.generated, r.finish_reason) for r in reqs]))
    return results


def test_running_ahead_gives_the_same_tokens_and_reasons():
    def add(s):
        return [s.add("a", list(range(20)), SamplingParams(max_tokens=12, stop_token_ids=(105,))),
                s.add("b", list(range(7)), SamplingParams(max_tokens=9)),
                s.add("c", list(range(33)), SamplingParams(max_tokens=20, stop_token_ids=(111, 103), ignore_eos=True))]
    (ex0, s0, want), (ex1, s1, got) = run_both(add, token_budget=16, prefill_chunk=8, max_running=3)
    assert got == want
    assert want[0] == ([100, 101, 102, 103, 104, 105], "stop") and want[1][1] == "length" and len(want[2][0]) == 20
    assert s0.steps_ahead == 0 and ex0.most_in_flight == 1
    assert s1.steps_ahead > 0 and ex1.most_in_flight == 2 and ex1.fed_from_device == s1.steps_ahead


def test_nothing_is_queued_ahead_while_a_prompt_waits_or_a_limit_is_near():
    ex = TwoPhaseExecutor()
    s = Scheduler(ex, token_budget=8, prefill_chunk=8, max_running=1)
    a = s.add("a", [1, 2, 3], SamplingParams(max_tokens=4))
    s.add("b", [1, 2, 3], SamplingParams(max_tokens=2))
    s.step()                                                     # a's prompt; b waits for the slot
    assert s._ahead is None and a.generated == [100]
    s.step(); s.step()
    assert s._ahead is None and s.steps_ahead == 0               # b still waits: every step is planned afresh
    s.run()
    assert s.steps_ahead == 1                                    # b, alone at last, had its second token queued
    # alone, a request is run ahead until its last token is queued
    ex = TwoPhaseExecutor()
    s = Scheduler(ex, token_budget=8, prefill_chunk=8)
    a = s.add("a", [1, 2, 3], SamplingParams(max_tokens=4))
    s.step()
    assert s._ahead is not None and a.generated == [100]         # token 2 of 4 is queued
    s.step()
    assert s._ahead is not None and a.generated == [100, 101]    # token 3 of 4 is queued
    s.step()
    assert s._ahead is not None and a.generated == [100, 101, 102]   # token 4, the last, is queued
    s.step()
    assert s._ahead is None and a.generated == [100, 101, 102, 103] and a.finish_reason == "length"
    assert s.idle and ex.log[-1] == [("a", 1, [0])] and len(ex.log) == 4


def test_penalties_keep_the_loop_waiting():
    def add(s):
        return [s.add("a", [1, 2, 3], SamplingParams(max_tokens=6, repetition_penalty=1.2))]
    (_, s0, want), (_, s1, got) = run_both(add)
    assert got == want and s1.steps_ahead == 0
