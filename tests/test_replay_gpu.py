"""Replay on the GPU against the plain implementation: every request whole, with the last 32 tokens one by
one, in portions of changing size, and mixed with other requests on a pool so small that pages are used
again; in 32-bit and in bfloat16, on both tiny configurations."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_mistral as pm
import tiny

pytestmark = pytest.mark.gpu

# Spread of the attention scores.  bfloat16 rounds q and k to 8 bits, which shifts a score of magnitude s by
# about s/256 and its softmax weight by as much, so the bfloat16 cases use scores a few units wide, where that
# noise stays well under the tolerance; faults of the cache and the batch logic are caught by the float32 cases,
# whose scores are spread wide, and single keys that must not be lost by the kernel tests.
SHARP = {"float32": 0.2, "bfloat16": 0.1}
LENGTHS = {"A": [5, 23, 40, 70, 33, 18, 64], "B": [1, 7, 31, 64, 47, 12, 80]}


@pytest.fixture(scope="module", params=[(c, d) for c in ("A", "B") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    name, dtype = request.param
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(tmp_path_factory.mktemp(f"model{name}{dtype}"), cfg, seed=11 if name == "A" else 23,
                              dtype=dtype, sharp=SHARP[dtype])
    requests = tiny.random_requests(cfg, LENGTHS[name], seed=5)
    pcfg, W = pm.read_model_folder(folder)
    want = {rid: pm.forward_logits(pcfg, W, toks) for rid, toks in requests.items()}
    return dict(name=name, dtype=dtype, cfg=cfg, folder=folder, requests=requests, want=want)


def run(case, schedule, tmp_path, slack_tokens=0):
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    tokens = schedule.max_live_tokens(case["requests"]) + slack_tokens
    engine = Engine.from_folder(case["folder"], EngineOptions(
        dtype=case["dtype"], cache_tokens=tokens, max_requests=4, max_step_tokens=max(tokens, 128),
        max_seq_len=max(tokens, 128)))
    replay(engine, schedule.lines(), tmp_path)
    engine.cache.check_invariants()
    assert not engine.cache.requests, "requests left live after the trace"
    assert all(g.pool.n_free == g.pool.n_pages for g in engine.cache.groups), "pages lost"
    got = tiny.read_rows(tmp_path, schedule, case["cfg"]["vocab_size"])
    return tiny.compare_rows(got, case["want"], tiny.TOL[case["dtype"]], f"{case['name']} {case['dtype']}")


def test_whole(case, tmp_path):
    run(case, tiny.schedule_whole(case["requests"]), tmp_path)


def test_last_32_one_by_one(case, tmp_path):
    run(case, tiny.schedule_tail(case["requests"], 32), tmp_path)


def test_portions_of_changing_size(case, tmp_path):
    run(case, tiny.schedule_portions(case["requests"]), tmp_path)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_mixed_with_page_reuse(case, tmp_path, seed):
    sched = tiny.schedule_mixed(case["requests"], seed=seed)
    total_pages = sum(-(-len(t) // 16) for t in case["requests"].values())
    pool_pages = sched.max_live_tokens(case["requests"]) // 16
    assert pool_pages < total_pages, "the pool must be smaller than what all requests need, so pages are reused"
    run(case, sched, tmp_path)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_a_careless_trace(case, tmp_path, seed):
    """Ids used again after their end, requests ended early, scattered wanted places, steps that want nothing."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    requests, sched = tiny.schedule_wild(case["cfg"], seed)
    by_name = {}
    tokens = 256                                   # four live requests of at most 100 tokens, each rounded up to 64
    engine = Engine.from_folder(case["folder"], EngineOptions(
        dtype=case["dtype"], cache_tokens=tokens, max_requests=4, max_step_tokens=256, max_seq_len=128))
    replay(engine, sched.lines(), tmp_path)
    engine.cache.check_invariants()
    got = tiny.read_rows(tmp_path, sched, case["cfg"]["vocab_size"])
    pcfg, W = pm.read_model_folder(case["folder"])
    worst = 0.0
    for (u, p), row in got.items():
        if u not in by_name:
            by_name[u] = pm.forward_logits(pcfg, W, requests[u]).numpy()
        ref = by_name[u]
        worst = max(worst, float(abs(row.astype("float64") - ref[p]).max()) / float(abs(ref).max()))
    assert got and worst <= tiny.TOL[case["dtype"]], f"error {worst:.3e} of the logit scale"


def test_trace_run_program(case, tmp_path):
    """The program itself, in a process of its own."""
    sched = tiny.schedule_mixed(case["requests"], seed=9)
    exe = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(exe), "--model", str(case["folder"]), "--dtype", case["dtype"], "--out", str(out),
         "--max-tokens", str(sched.max_live_tokens(case["requests"]))],
        input="\n".join(sched.lines()) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(sched.steps))]
    got = tiny.read_rows(out, sched, case["cfg"]["vocab_size"])
    tiny.compare_rows(got, case["want"], tiny.TOL[case["dtype"]], "trace_run")
