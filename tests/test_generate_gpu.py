"""Generation through the Python entry point and the command line, long decoding, and the first tokens of a
sequence, against the plain implementation."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_mistral as pm
import tiny

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module", params=[("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def model(request, tmp_path_factory):
    name, dtype = request.param
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(tmp_path_factory.mktemp(f"gen{name}{dtype}"), cfg, seed=31, dtype=dtype,
                              sharp=0.2 if dtype == "float32" else 0.1)
    pcfg, W = pm.read_model_folder(folder)
    return dict(name=name, dtype=dtype, cfg=cfg, folder=folder, pcfg=pcfg, W=W)


def check_greedy(model, prompts, outs, n_new):
    """Each generated token must be the plain implementation's argmax given what came before it (in bfloat16:
    within the tolerance of the best logit, since near-ties may fall either way)."""
    for prompt, out in zip(prompts, outs):
        assert len(out) == n_new
        toks = list(prompt)
        for t in out:
            logits = pm.forward_logits(model["pcfg"], model["W"], toks)[-1]
            if model["dtype"] == "float32":
                assert t == pm.argmax_lowest(logits), "greedy token differs from the plain implementation"
            else:
                gap = float(logits.max() - logits[t]) / float(logits.abs().max())
                assert gap <= 2 * tiny.TOL["bfloat16"], f"token {t} is {gap:.3f} of the scale below the best logit"
            toks.append(t)


def test_greedy_generation_matches(model):
    from flambeau_b200 import generate
    lengths = [5, 23, 40] if model["name"] == "A" else [1, 7, 31, 64]
    prompts = list(tiny.random_requests(model["cfg"], lengths, seed=8).values())
    outs = generate(model["folder"], prompts, max_tokens=8, temperature=0.0, dtype=model["dtype"],
                    prefill_chunk_tokens=8, prefill_ubatch=24, inflight_slots=4)
    check_greedy(model, prompts, outs, 8)


def test_generation_under_page_pressure_gives_the_same_tokens(model):
    """So few pages that requests are preempted and fed again: the tokens must not change."""
    from flambeau_b200.engine.generate import Generator
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.sampling.params import SamplingParams
    if model["dtype"] != "float32":
        pytest.skip("token-for-token equality is a float32 property")
    # A pool that the requests outgrow while they decode.  Without a window every request keeps growing.  Under
    # a window a request holds two pages at most, so the prompts are short enough to be admitted side by side on
    # one page each, and the pool has five pages for the eight they come to need.
    windowed = model["cfg"]["sliding_window"] is not None
    lengths, tight_tokens = ([5, 9, 7, 12], 80) if windowed else ([20, 33, 18, 27], 112)
    prompts = list(tiny.random_requests(model["cfg"], lengths, seed=9).values())
    params = SamplingParams(max_tokens=30)
    roomy = Engine.from_folder(model["folder"], EngineOptions(dtype="float32", cache_tokens=512, max_requests=4,
                                                              max_step_tokens=64, max_seq_len=128))
    want = Generator(roomy, prefill_chunk_tokens=16).generate(prompts, params)
    tight = Engine.from_folder(model["folder"], EngineOptions(dtype="float32", cache_tokens=tight_tokens, max_requests=4,
                                                              max_step_tokens=64, max_seq_len=128))
    gen = Generator(tight, prefill_chunk_tokens=16)
    got = gen.generate(prompts, params)
    assert got == want
    sched = gen.last_scheduler
    assert sum(r.preemptions for r in sched.finished) > 0, "the pool was meant to be too small"
    assert all(r.finish_reason == "length" for r in sched.finished)
    tight.cache.check_invariants()
    assert not tight.cache.requests


def test_running_ahead_changes_no_token(model):
    """Decode steps queued before the host has read the tokens of the step before (their ids fed on the device),
    against the loop that waits every step: stop tokens in mid-flight, unequal limits, draws and greedy rows."""
    from flambeau_b200.engine.generate import Generator
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.sampling.params import SamplingParams
    prompts = list(tiny.random_requests(model["cfg"], [9, 30, 4, 17], seed=21).values())
    engine = Engine.from_folder(model["folder"], EngineOptions(dtype=model["dtype"], cache_tokens=512, max_requests=4,
                                                               max_step_tokens=64, max_seq_len=128))
    free = Generator(engine, prefill_chunk_tokens=16, run_ahead=False).generate(
        prompts, [SamplingParams(max_tokens=24, temperature=0.9, seed=3 + i) for i in range(4)])
    # stop tokens taken from what the requests really generate, so that they stop in the middle of the run
    params = [SamplingParams(max_tokens=24, temperature=0.9, seed=3, stop_token_ids=(free[0][7],)),
              SamplingParams(max_tokens=13, temperature=0.9, seed=4),
              SamplingParams(max_tokens=24, temperature=0.0, stop_token_ids=(free[2][3], free[2][15])),
              SamplingParams(max_tokens=24, temperature=0.9, seed=6, repetition_penalty=1.0)]
    waiting = Generator(engine, prefill_chunk_tokens=16, run_ahead=False)
    want = waiting.generate(prompts, params)
    ahead = Generator(engine, prefill_chunk_tokens=16, run_ahead=True)
    got = ahead.generate(prompts, params)
    assert got == want
    assert ahead.last_scheduler.steps_ahead > 5, "steps were meant to be queued ahead"
    assert waiting.last_scheduler.steps_ahead == 0
    assert [r.finish_reason for r in ahead.last_scheduler.finished] == \
           [r.finish_reason for r in waiting.last_scheduler.finished]
    assert len(got[0]) < 24 and len(got[1]) == 13
    engine.cache.check_invariants()
    assert not engine.cache.requests
    # a request with penalties needs its tokens on the host: nothing is queued ahead, the tokens agree all the same
    pen = [SamplingParams(max_tokens=10, temperature=0.7, seed=9, repetition_penalty=1.3)] * 4
    a = Generator(engine, prefill_chunk_tokens=16, run_ahead=True)
    assert a.generate(prompts, pen) == waiting.generate(prompts, pen)
    assert a.last_scheduler.steps_ahead == 0


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(model):
    from flambeau_b200 import generate
    prompts = list(tiny.random_requests(model["cfg"], [6, 19, 11], seed=10).values())
    kw = dict(max_tokens=6, temperature=0.8, seed=5, dtype=model["dtype"], prefill_chunk_tokens=8)
    a = generate(model["folder"], prompts, **kw)
    b = generate(model["folder"], prompts, **kw)
    assert a == b, "same seed, same tokens"
    c = generate(model["folder"], prompts, **{**kw, "seed": 6})
    assert c != a
    if model["dtype"] == "float32":
        alone = generate(model["folder"], [prompts[1]], **{**kw, "seed": 6})      # request 1 of seed 5 draws with 5+1
        assert alone[0] == a[1], "a request's draws do not depend on what shares its batches"
    d = generate(model["folder"], prompts, **{**kw, "top_k": 1})
    g = generate(model["folder"], prompts, **{**kw, "temperature": 0.0})
    assert d == g, "top_k = 1 is greedy"


def test_long_decoding_and_first_tokens(model, tmp_path):
    """One token a step from the very first token on, for far longer than the window and several pages."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    reqs = tiny.random_requests(model["cfg"], [150], seed=12)
    sched = tiny.schedule_tail(reqs, tail=149)                    # position 0 alone, then 149 single tokens
    engine = Engine.from_folder(model["folder"], EngineOptions(dtype=model["dtype"], cache_tokens=192, max_requests=2,
                                                               max_step_tokens=16, max_seq_len=192))
    replay(engine, sched.lines(), tmp_path)
    assert engine.graph_replays > 100, "single-token steps are replayed from a captured graph"
    want = {rid: pm.forward_logits(model["pcfg"], model["W"], toks) for rid, toks in reqs.items()}
    got = tiny.read_rows(tmp_path, sched, model["cfg"]["vocab_size"])
    tiny.compare_rows(got, want, tiny.TOL[model["dtype"]], f"long decode {model['name']} {model['dtype']}")


def test_context_cap_ends_a_request(model):
    """--ctx-cap: a request never holds more tokens than that, generated ones included."""
    from flambeau_b200 import generate
    prompts = [list(range(1, 41)), list(range(1, 11)), list(range(1, 60))]
    outs = generate(model["folder"], prompts, max_tokens=20, dtype=model["dtype"], ctx_cap=48, inflight_slots=3)
    assert [len(o) for o in outs] == [8, 20, 0]
    free = generate(model["folder"], prompts[:2], max_tokens=20, dtype=model["dtype"], inflight_slots=2)
    if model["dtype"] == "float32":
        assert outs[0] == free[0][:8] and outs[1] == free[1]


def test_command_line_infer(model):
    prompts = list(tiny.random_requests(model["cfg"], [9, 4], seed=13).values())
    cmd = [sys.executable, str(ROOT / "bin" / "flambeau"), "infer", "--model", str(model["folder"]), "--max-tokens", "5",
           "--dtype", model["dtype"]]
    for p in prompts:
        cmd += ["--prompt", ",".join(map(str, p))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    outs = [[int(t) for t in line.split(",")] for line in proc.stdout.strip().splitlines()]
    check_greedy(model, prompts, outs, 5)


def test_errors_are_raised_before_anything_runs(model):
    from flambeau_b200.cache.pages import OutOfPages
    from flambeau_b200.engine.batch import BatchError
    from flambeau_b200.engine.step import Engine, EngineOptions
    e = Engine.from_folder(model["folder"], EngineOptions(dtype=model["dtype"], cache_tokens=32, max_requests=2,
                                                          max_step_tokens=64, max_seq_len=64))
    with pytest.raises(OutOfPages):
        e.step([("a", list(range(40)), [])])
    assert not e.cache.requests and e.cache.free_pages() == [2]
    with pytest.raises(BatchError):
        e.step([("a", [model["cfg"]["vocab_size"]], [0])])
    with pytest.raises(BatchError):
        e.step([("a", [1, 2], [2])])
    logits = e.step([("a", [1, 2, 3], [2])], end=["a"])
    assert logits.shape == (1, model["cfg"]["vocab_size"]) and torch.isfinite(logits).all()
    assert not e.cache.requests


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_request_comes_back_from_a_snapshot(name, tmp_path):
    """Thirty tokens in, snapshot, release, other requests through the same pages, restore under another id,
    ten more tokens: the logits are those of the request that never left, bit for bit."""
    from flambeau_b200.engine.batch import Entry
    from flambeau_b200.engine.step import Engine, EngineOptions
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(tmp_path / "m", cfg, seed=6, dtype="float32")
    toks = tiny.random_requests(cfg, [40, 25], seed=12)
    a, other = toks["r0"], toks["r1"]
    engine = Engine.from_folder(folder, EngineOptions(dtype="float32", cache_tokens=96, max_requests=2,
                                                      max_step_tokens=64, max_seq_len=64, cuda_graphs=False))
    engine.step([Entry("stay", a[:30], [])])
    want = [engine.step([Entry("stay", [t], [0])]).clone() for t in a[30:]]
    engine.finish("stay")
    engine.step([Entry("go", a[:30], [])])
    snap = engine.snapshot("go")
    assert snap.length == 30 and snap.nbytes() > 0
    engine.finish("go")
    engine.step([Entry("other", other, [len(other) - 1])], end=["other"])      # the freed pages are written over
    engine.step([Entry("other2", other[:9], [])])                               # and some are held by someone else
    engine.restore("back", snap)
    got = [engine.step([Entry("back", [t], [0])]).clone() for t in a[30:]]
    engine.runtime.check_status("restore")
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    engine.finish("back")
    engine.finish("other2")
    engine.cache.check_invariants()
    assert not engine.cache.requests
