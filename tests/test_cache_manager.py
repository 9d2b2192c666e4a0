"""The page pool and the cache manager on the CPU: no page lost, held twice or freed twice, under random
orders of requests; windowed release; fixed-size state slots."""
import random

import pytest
import torch

from flambeau_b200.cache.manager import CacheManager, CallPlan
from flambeau_b200.cache.pages import Books, OutOfPages, PageError
from flambeau_b200.parts.base import KVRequirement, StateRequirement


class PagePool:
    """A pool on its own, driven through the books (one group, one request slot per held page, pages of one
    token): what the cache manager's groups are made of."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = int(n_pages)
        # one request slot per possible holder of a single page; page_size 1 makes a token a page
        self._books = Books([self.n_pages], [0], 1, self.n_pages + 1, self.n_pages)
        self._holder: dict = {}              # page id -> slot that holds it

    @property
    def n_free(self) -> int:
        return self._books.free_pages()[0]

    @property
    def n_held(self) -> int:
        return self.n_pages - self.n_free

    def take(self, count: int) -> list:
        """`count` page ids, or OutOfPages with nothing taken."""
        if count < 0:
            raise ValueError("negative page count")
        if count > self.n_free:
            raise OutOfPages(count, self.n_free, self.n_pages)
        out = []
        for _ in range(count):
            slot = self._books.admit()
            self._books.reserve_all([slot], [1])
            page = self._books.pages(slot, 0)[0]
            self._holder[page] = slot
            out.append(page)
        return out

    def give_back(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages:
                raise PageError(f"page id {p} is outside the pool of {self.n_pages}")
            slot = self._holder.pop(p, None)
            if slot is None:
                raise PageError(f"page {p} is given back but is not held")
            self._books.release(slot)

    def is_held(self, page: int) -> bool:
        return self._books.is_held(0, page)


def test_pool_is_fifo_and_all_or_nothing():
    pool = PagePool(4)
    a = pool.take(3)
    assert a == [0, 1, 2] and pool.n_free == 1
    with pytest.raises(OutOfPages):
        pool.take(2)
    assert pool.n_free == 1                      # nothing was taken
    pool.give_back([1])
    assert pool.take(2) == [3, 1]                # reused in the order of return
    with pytest.raises(PageError):
        pool.give_back([0, 0])                   # freed twice
    with pytest.raises(PageError):
        pool.give_back([7])


def manager(window=0, tokens=256, layers=2, max_requests=4, state=False, max_seq_len=None):
    plans = [CallPlan(kv=KVRequirement(2, 16, window), state=StateRequirement((3,)) if state else None)
             for _ in range(layers)]
    return CacheManager(plans, max_tokens=tokens, page_size=16, max_requests=max_requests, device="cpu",
                        dtype=torch.float32, max_seq_len=max_seq_len or tokens)


def test_groups_follow_requirements():
    plans = [CallPlan(kv=KVRequirement(2, 16, 0)), CallPlan(kv=KVRequirement(2, 16, 8)),
             CallPlan(kv=KVRequirement(2, 16, 0)), CallPlan(kv=None, state=StateRequirement((5,))),
             CallPlan(kv=KVRequirement(2, 16, 0), cache_from=0)]
    cm = CacheManager(plans, max_tokens=64, page_size=16, max_requests=2, device="cpu", dtype=torch.float32)
    assert cm.n_groups == 2
    assert cm.group_of_call[0] == cm.group_of_call[2] == cm.group_of_call[4] != cm.group_of_call[1]
    assert 3 not in cm.group_of_call and cm.state[3].shape == (2, 5)
    v = cm.view(4, [None, None])
    assert not v.writable and v.k_pool is cm.groups[cm.group_of_call[0]].k[0]
    assert cm.view(2, [None, None]).writable
    with pytest.raises(ValueError):
        CacheManager([CallPlan(kv=None), CallPlan(kv=KVRequirement(1, 8), cache_from=0)], max_tokens=64,
                     page_size=16, max_requests=1, device="cpu", dtype=torch.float32)


def test_reserve_is_all_or_nothing_and_release_returns_everything():
    cm = manager(tokens=64)                      # 4 pages
    cm.admit("a")
    cm.reserve("a", 40)                          # 3 pages
    cm.commit("a", 40)
    cm.admit("b")
    assert not cm.can_reserve([("b", 17)])
    with pytest.raises(OutOfPages):
        cm.reserve("b", 17)
    assert cm.free_pages() == [1]
    cm.reserve("b", 16)
    cm.commit("b", 16)
    cm.check_invariants()
    cm.release("a")
    cm.release("b")
    assert cm.free_pages() == [4] and not cm.requests
    with pytest.raises(KeyError):
        cm.release("a")


def test_window_gives_pages_back_as_they_die():
    cm = manager(window=16, tokens=64, max_seq_len=128)
    cm.admit("a")
    held = []
    for _ in range(10):                          # 100 tokens through a 4-page pool
        cm.reserve("a", 10)
        cm.commit("a", 10)
        cm.check_invariants()
        held.append(4 - cm.free_pages()[0])
    assert max(held) <= 3
    rec = cm.requests["a"]
    first_live = rec.length - 16 + 1
    for j, p in enumerate(rec.pages[0]):
        assert (p < 0) == ((j + 1) * 16 <= first_live), "exactly the pages wholly below the window are given back"
    assert cm.first_live_page("a", 0) == first_live // 16
    cm.release("a")
    assert cm.free_pages() == [4]


def test_commit_beyond_reservation_is_an_error():
    cm = manager()
    cm.admit("a")
    cm.reserve("a", 5)
    with pytest.raises(PageError):
        cm.commit("a", 6)


def test_state_slots_are_zeroed_on_admission_and_reused():
    cm = manager(state=True, max_requests=2)
    a = cm.admit("a")
    cm.state[0][a.slot] += 5.0
    b = cm.admit("b")
    assert a.slot != b.slot
    with pytest.raises(PageError):
        cm.admit("c")
    cm.release("a")
    c = cm.admit("c")
    assert c.slot == a.slot and float(cm.state[0][c.slot].abs().sum()) == 0.0
    assert cm.state_bytes_per_request() == 2 * 3 * 4


@pytest.mark.parametrize("window", [0, 16, 40])
@pytest.mark.parametrize("seed", range(5))
def test_random_orders_never_lose_or_double_a_page(window, seed):
    rng = random.Random(seed)
    cm = manager(window=window, tokens=192, max_requests=4)
    live, next_id = {}, 0
    for _ in range(400):
        r = rng.random()
        if r < 0.25 and cm.has_slot():
            cm.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif r < 0.85 and live:
            rid = rng.choice(list(live))
            k = rng.choice([1, 1, 1, 2, 5, 17, 33])
            if cm.can_reserve([(rid, k)]) and cm.length(rid) + k <= 192:
                before = cm.free_pages()
                cm.reserve(rid, k)
                cm.commit(rid, k)
                live[rid] += k
                assert cm.length(rid) == live[rid]
                if window == 0:
                    assert before[0] - cm.free_pages()[0] == -(-live[rid] // 16) - -(-(live[rid] - k) // 16)
            else:
                free = cm.free_pages()
                if not cm.can_reserve([(rid, k)]):
                    with pytest.raises(OutOfPages):
                        cm.reserve(rid, k)
                    assert cm.free_pages() == free
        elif live:
            rid = rng.choice(list(live))
            cm.release(rid)
            del live[rid]
        cm.check_invariants()
        held = sum(sum(1 for p in rec.pages[0] if p >= 0) for rec in cm.requests.values())
        assert held + cm.free_pages()[0] == cm.groups[0].pool.n_pages
    cm.release_all()
    assert cm.free_pages() == [12]


def test_a_reader_may_not_look_further_back_than_the_cache_it_reads_keeps():
    """Pages are given back by the owner's window; a call that reads that cache with no window, or a wider one,
    would ask for keys whose pages are gone."""
    def build(owner_window, reader_window):
        return CacheManager([CallPlan(kv=KVRequirement(2, 16, owner_window)),
                             CallPlan(kv=KVRequirement(2, 16, reader_window), cache_from=0)],
                            max_tokens=64, page_size=16, max_requests=1, device="cpu", dtype=torch.float32)
    for owner, reader in ((16, 0), (16, 32)):
        with pytest.raises(ValueError, match="keeps only"):
            build(owner, reader)
    for owner, reader in ((0, 0), (0, 8), (32, 32), (32, 8)):
        build(owner, reader)


def test_a_windowed_request_outlives_its_table_row():
    """A block-table row holds live pages only, so a request under a window runs on far past the number of
    tokens that the row's columns could address from position 0."""
    plans = [CallPlan(kv=KVRequirement(1, 8, 24))]
    cm = CacheManager(plans, max_tokens=128, page_size=8, max_requests=2, device="cpu", dtype=torch.float32,
                      max_seq_len=100000, max_step_tokens=16)
    assert cm.table_pages == -(-(24 + 16) // 8) + 2
    cm.admit("a")
    for _ in range(300):                          # 4,800 tokens through a row of 7 columns and a pool of 16 pages
        cm.reserve("a", 16)
        live = [p for p in cm.requests["a"].pages[0] if p >= 0]
        assert len(live) <= cm.table_pages
        cm.commit("a", 16)
        cm.check_invariants()
    assert cm.length("a") == 4800 and cm.first_live_page("a", 0) == (4800 - 24 + 1) // 8


@pytest.mark.parametrize("window", [0, 24])
def test_snapshot_and_restore_bring_a_request_back(window):
    """What a request holds goes to the host and comes back into other pages and another slot: same length, same
    first live page, same contents by logical page, same state; all or nothing when pages are short."""
    plans = [CallPlan(kv=KVRequirement(2, 4, window), state=StateRequirement((3,))), CallPlan(kv=KVRequirement(2, 4, window))]
    cm = CacheManager(plans, max_tokens=128, page_size=8, max_requests=4, device="cpu", dtype=torch.float32,
                      max_seq_len=512)
    g = cm.groups[0]
    for t in list(g.k.values()) + list(g.v.values()):
        t.copy_(torch.arange(t.numel(), dtype=torch.float32).view_as(t))     # every element names its place
    cm.admit("a")
    for _ in range(9):
        cm.reserve("a", 7)
        cm.commit("a", 7)                                                      # 63 tokens; under the window pages go back
    cm.state[0][cm.requests["a"].slot] = torch.tensor([1.0, 2.0, 3.0])
    before_pages = [p for p in cm.requests["a"].pages[0]]
    live = [p for p in before_pages if p >= 0]
    snap = cm.snapshot("a")
    assert snap.length == 63 and snap.first_pages == [cm.first_live_page("a", 0)]
    assert snap.k[0].shape[0] == len(live) and torch.equal(snap.k[1], g.k[1][live])
    cm.release("a")
    cm.admit("other")
    cm.reserve("other", 20)                                                    # takes the pages that came back first
    cm.commit("other", 20)
    for t in list(g.k.values()) + list(g.v.values()):
        t.zero_()
    cm.restore("b", snap)
    cm.check_invariants()
    rec = cm.requests["b"]
    assert rec.length == 63 and cm.first_live_page("b", 0) == snap.first_pages[0]
    after = [p for p in rec.pages[0]]
    assert [p < 0 for p in after] == [p < 0 for p in before_pages]
    now_live = [p for p in after if p >= 0]
    assert now_live != live, "the request came back into other pages"
    for c in (0, 1):
        assert torch.equal(g.k[c][now_live], snap.k[c]) and torch.equal(g.v[c][now_live], snap.v[c])
    assert cm.state[0][rec.slot].tolist() == [1.0, 2.0, 3.0]
    cm.reserve("b", 5)                                                         # and goes on
    cm.commit("b", 5)
    assert cm.length("b") == 68
    with pytest.raises(PageError):
        cm.restore("b", snap)                                                  # already live
    free = cm.free_pages()
    big = cm.snapshot("b")
    cm.admit("hog")
    cm.reserve("hog", free[0] * 8)
    with pytest.raises(OutOfPages):
        cm.restore("c", big)
    assert cm.free_pages() == [0] and "c" not in cm.requests
    cm.check_invariants()
