"""The packing of a step's descriptor (C++ host code) on the CPU, against a restatement in Python: rows, sequences,
wanted rows and block tables for random mixes of portions and single tokens, over groups with and without a
window, while pages are released and reused; and what it refuses."""
import random

import numpy as np
import pytest
import torch

from flambeau_b200.cache.manager import CacheManager, CallPlan
from flambeau_b200.engine.batch import BatchBuffers, BatchError, Entry
from flambeau_b200.parts.base import KVRequirement

VOCAB = 500


def make(tokens=256, window=24, max_requests=4, page_size=8, max_step=64):
    cache = CacheManager([CallPlan(kv=KVRequirement(1, 8, 0)), CallPlan(kv=KVRequirement(2, 8, window))],
                         max_tokens=tokens, page_size=page_size, max_requests=max_requests, device="cpu",
                         dtype=torch.float32, max_seq_len=tokens, max_step_tokens=max_step)
    buffers = BatchBuffers(torch.device("cpu"), max_step, max_requests, cache.n_groups, cache.table_pages)
    return cache, buffers


def expected(cache, entries):
    rows = dict(tok=[], pos=[], seq=[], out=[])
    seqs = dict(start=[], qlen=[], pos0=[], slot=[])
    at = 0
    for s, e in enumerate(entries):
        rec = cache.requests[e.request_id]
        seqs["start"].append(at); seqs["qlen"].append(len(e.tokens)); seqs["pos0"].append(rec.length)
        seqs["slot"].append(rec.slot)
        for j, t in enumerate(e.tokens):
            rows["tok"].append(t); rows["pos"].append(rec.length + j); rows["seq"].append(s)
        rows["out"] += [at + w for w in e.want]
        at += len(e.tokens)
    return rows, seqs


@pytest.mark.parametrize("seed", range(8))
def test_descriptor_of_random_steps(seed):
    rng = random.Random(seed)
    cache, buffers = make()
    live, done_ids = {}, 0
    for step in range(60):
        while len(live) < 4 and rng.random() < 0.6:
            rid = f"r{done_ids}"
            done_ids += 1
            cache.admit(rid)
            live[rid] = 0
        if not live:
            continue
        chosen = [rid for rid in live if rng.random() < 0.8] or [next(iter(live))]
        rng.shuffle(chosen)
        entries, left = [], 64
        for rid in chosen:
            k = min(rng.choice([1, 1, 1, 2, 5, 13, 30]), left, 256 - 8 - cache.length(rid))
            if k <= 0:
                continue
            if not cache.can_reserve([(e.request_id, len(e.tokens)) for e in entries] + [(rid, k)]):
                continue
            toks = [rng.randrange(VOCAB) for _ in range(k)]
            want = sorted(rng.sample(range(k), rng.randint(0, min(k, 3))))
            entries.append(Entry(rid, toks, want))
            left -= k
        if not entries:
            victim = rng.choice(list(live))
            cache.release(victim)
            del live[victim]
            continue
        cache.reserve_all([(e.request_id, len(e.tokens)) for e in entries])
        b = buffers.build(entries, cache, VOCAB)
        rows, seqs = expected(cache, entries)
        n, S = len(rows["tok"]), len(entries)
        assert (b.n_tokens, b.n_seqs, b.n_out) == (n, S, len(rows["out"]))
        assert b.token_ids[:n].tolist() == rows["tok"] and b.positions[:n].tolist() == rows["pos"]
        assert b.row_seq[:n].tolist() == rows["seq"] and b.out_rows[:b.n_out].tolist() == rows["out"]
        assert b.seq_q_start_d[:S].tolist() == seqs["start"] == b.seq_q_start
        assert b.seq_q_len_d[:S].tolist() == seqs["qlen"] == b.seq_q_len
        assert b.seq_pos_start_d[:S].tolist() == seqs["pos0"] == b.seq_pos_start
        assert b.seq_slot_d[:S].tolist() == seqs["slot"] == b.seq_slot
        assert b.max_q_len == max(seqs["qlen"])
        assert b.multi_seqs_d[:b.n_multi].tolist() == [s for s, q in enumerate(seqs["qlen"]) if q > 1]
        assert b.max_kv_len >= max(p + q for p, q in zip(seqs["pos0"], seqs["qlen"]))
        for gi in range(cache.n_groups):
            for s, e in enumerate(entries):
                pages = list(cache.table_row(e.request_id, gi))      # by logical page, -1 = given back
                base = cache.first_live_page(e.request_id, gi)
                got = b.tables[gi][s].tolist()
                # the row holds the live pages only, from the first live page on
                assert all(p < 0 for p in pages[:base]) and all(p >= 0 for p in pages[base:])
                assert int(b.table_bases[gi][s]) == base
                assert got[:len(pages) - base] == pages[base:], f"group {gi} sequence {s}"
                assert all(p == -1 for p in got[len(pages) - base:]), "what an earlier request left in the row"
                # every position a query of this step can see has a page
                window = cache.groups[gi].req.window
                first_q, last_q = seqs["pos0"][s], seqs["pos0"][s] + seqs["qlen"][s] - 1
                lo = max(0, first_q - window + 1) if window else 0
                assert all(got[p // 8 - base] >= 0 for p in range(lo, last_q + 1))
        cache.commit_all([(e.request_id, len(e.tokens)) for e in entries])
        cache.check_invariants()
        for e in entries:
            live[e.request_id] += len(e.tokens)
            if rng.random() < 0.1:
                cache.release(e.request_id)
                del live[e.request_id]
    cache.release_all()
    assert cache.free_pages() == [g.pool.n_pages for g in cache.groups]


def test_what_the_packing_refuses():
    cache, buffers = make(max_step=16)
    for rid in "ab":
        cache.admit(rid)
    cache.reserve("a", 4)
    cache.reserve("b", 4)
    with pytest.raises(BatchError, match="at least one entry"):
        buffers.build([], cache, VOCAB)
    with pytest.raises(BatchError, match="twice"):
        buffers.build([Entry("a", [1]), Entry("a", [2])], cache, VOCAB)
    with pytest.raises(BatchError, match="no tokens"):
        buffers.build([Entry("a", [])], cache, VOCAB)
    with pytest.raises(BatchError, match="outside"):
        buffers.build([Entry("a", [1, 2], [2])], cache, VOCAB)
    with pytest.raises(BatchError, match="token id"):
        buffers.build([Entry("a", [VOCAB])], cache, VOCAB)
    with pytest.raises(BatchError, match="token id"):
        buffers.build([Entry("a", [-1])], cache, VOCAB)
    with pytest.raises(BatchError):
        buffers.build([Entry("a", [1, 2, 3, 4, 5])], cache, VOCAB)         # one token more than was reserved
    with pytest.raises(KeyError):
        buffers.build([Entry("zzz", [1])], cache, VOCAB)
    cache.reserve("a", 20)
    with pytest.raises(BatchError):
        buffers.build([Entry("a", list(range(17)))], cache, VOCAB)          # more rows than a step may bring
    b = buffers.build([Entry("a", [1, 2, 3, 4], [3]), Entry("b", [5], [0])], cache, VOCAB)   # still usable afterwards
    assert (b.n_tokens, b.n_out) == (5, 2) and b.out_rows[:2].tolist() == [3, 4]
