"""The workloads that are measured, each through the engine's own calls.

  decode_device     engine.step + on-device sampling with fixed tokens, timed with CUDA events
  decode_e2e        the scheduler's loop (what generate() runs): host token ids in and out every step
  prefill_step      one bare engine.step of a whole prompt
  time_to_first     a prompt through Generator.generate with max_tokens = 1: the reference's prefill figure
                    (prompt tokens / time to the first token, doc/PERF_MATRIX.md:4-8)
  kernel_sections   one eager step under the section timer, folded into kernel classes
  mixed_requests    many requests of seeded lengths through the scheduler, with per-request first-token and
                    last-token times (scripts/bench/bench_mixed_sustained.py is the reference's counterpart)
  step_host_device  host time against device time of one mixed step
  attention_check   the decode attention of one layer against a float32 softmax over the same pages

Decoding is measured on requests whose cache is laid out by the cache manager as a real request of that length
leaves it (pages taken and, under a window, given back) but filled with random numbers instead of the result
of a prefill ("seated" requests)."""
from __future__ import annotations

import os
import random
import statistics
import sys
import time

import torch

from ..engine.batch import Entry
from ..engine.generate import EngineExecutor, Generator
from ..engine.scheduler import Request, Scheduler
from ..kernels import library, ops
from ..sampling.params import SamplingParams
from . import work
from .timers import SectionTimer


def randomise_cache(engine) -> None:
    """Random keys and values stand in for a real prefill."""
    for g in engine.cache.groups:
        for c in g.owners:
            g.k[c].normal_(0.0, 1.0)
            g.v[c].normal_(0.0, 1.0)


def seat(engine, contexts, prefix: str = "seq") -> list:
    """One request per entry of `contexts` whose cache holds context - 1 tokens (the books only)."""
    engine.cache.release_all()
    ids = []
    for i, context in enumerate(contexts):
        rid = f"{prefix}{i}"
        engine.cache.admit(rid)
        left = context - 1
        while left > 0:
            k = min(left, 256)
            engine.cache.reserve(rid, k)
            engine.cache.commit(rid, k)
            left -= k
        ids.append(rid)
    return ids


def decode_device(engine, batch: int, context: int, steps: int, warmup: int, gen) -> tuple:
    """(milliseconds per step, launches per step) of engine.step + on-device sampling with fixed input tokens."""
    ids = seat(engine, [context] * batch)
    vocab = engine.model.vocab_size
    tok = torch.randint(0, vocab, (batch,), generator=gen).tolist()
    entries = [Entry(r, [t], [0]) for r, t in zip(ids, tok)]
    chosen = torch.zeros(batch, dtype=torch.int32, device=engine.runtime.device)
    for _ in range(warmup):
        ops.sample(engine.step(entries), chosen, n=batch)
    torch.cuda.synchronize()
    l0 = library.LAUNCHES[0]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        ops.sample(engine.step(entries), chosen, n=batch)
    t1.record()
    torch.cuda.synchronize()
    engine.runtime.check_status("decode")
    return t0.elapsed_time(t1) / steps, (library.LAUNCHES[0] - l0) / steps


def decode_e2e(engine, batch: int, context: int, steps: int, warmup: int, gen) -> tuple:
    """(tokens a second, host-to-device bytes a step, device-to-host bytes a step) through the scheduler loop
    that generate() runs: host ids in, host ids out."""
    ids = seat(engine, [context] * batch)
    vocab = engine.model.vocab_size
    ex = EngineExecutor(engine)
    sched = Scheduler(ex, token_budget=max(batch, 1), prefill_chunk=512, max_running=batch)
    for i, rid in enumerate(ids):
        r = Request(rid, prompt=[0] * (context - 1), params=SamplingParams(max_tokens=steps + warmup + 8),
                    generated=[int(torch.randint(0, vocab, (1,), generator=gen))], arrival=i)
        r.fed = context - 1
        sched.running.append(r)
    ahead = sched.run_ahead

    def run_steps(n: int) -> None:
        # the scheduler queues each step before it reads the tokens of the one before; the last step of a
        # region queues nothing, so the region holds exactly the device work of the tokens it delivers
        for i in range(n):
            sched.run_ahead = ahead and i < n - 1
            assert len(sched.step()) == batch

    run_steps(warmup)
    torch.cuda.synchronize()
    h0, d0 = ex.h2d_bytes, ex.d2h_bytes
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    t0.record()
    run_steps(steps)
    t1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - w0
    ms = max(t0.elapsed_time(t1), wall * 1e3)
    for rid in ids:
        engine.cache.release(rid)
    return batch * steps / (ms / 1e3), (ex.h2d_bytes - h0) / steps, (ex.d2h_bytes - d0) / steps


def prefill_step(engine, tokens: int, gen, reps: int = 5, warmup: int = 3) -> float:
    """Median milliseconds of one engine.step that brings a whole prompt of `tokens` tokens."""
    engine.cache.release_all()
    toks = torch.randint(0, engine.model.vocab_size, (tokens,), generator=gen).tolist()
    times = []
    for i in range(warmup + reps):
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        engine.step([Entry("prompt", toks, [tokens - 1])], end=["prompt"])
        t1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(t0.elapsed_time(t1))
    engine.runtime.check_status("prefill")
    return statistics.median(times)


def time_to_first(engine, tokens: int, chunk: int, gen, reps: int = 3, warmup: int = 2) -> float:
    """Median milliseconds from handing a prompt of `tokens` tokens to Generator.generate to having its first
    token on the host, the prompt cut into portions of `chunk` by the scheduler."""
    engine.cache.release_all()
    toks = torch.randint(0, engine.model.vocab_size, (tokens,), generator=gen).tolist()
    g = Generator(engine, prefill_chunk_tokens=chunk, prefill_ubatch=chunk)
    times = []
    for i in range(warmup + reps):
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        out = g.generate([toks], SamplingParams(max_tokens=1))
        times.append((time.perf_counter() - w0) * 1e3)
        assert len(out[0]) == 1
    return statistics.median(times[warmup:])


def classify(cfg, what: str, note) -> str:
    """The kernel class of a launcher call."""
    s = work.sizes(cfg)
    if what.startswith("gemm"):
        matrix = tuple(note[1:]) if note else None
        names = {(s["qw"] + 2 * s["kvw"], s["H"]): "qkv_proj", (s["H"], s["qw"]): "o_proj",
                 (2 * s["I"], s["H"]): "gate_up_proj", (s["H"], s["I"]): "down_proj", (s["V"], s["H"]): "lm_head"}
        return names.get(matrix, what)
    return {"add_rms_norm": "add_norm", "rope_kv_write": "rotary_cache_write", "paged_attention_mma": "attention",
            "paged_attention_simt": "attention"}.get(what, what)


class Sections(dict):
    """class -> (launches per step, milliseconds per step), and in `ops` the launcher calls that were seen."""
    ops: frozenset = frozenset()


def kernel_sections(engine, entries, cfg, reps: int = 3, end=(), ahead_ms: float = 40.0) -> dict:
    """class -> (launches per step, milliseconds per step) of one eager step of `entries`.  The step is run
    `reps + 1` times in a row, so the entries must stay valid: decoded tokens are; a whole prompt is when `end`
    names its request, which then gives back what it holds after every run."""
    was = engine.use_graphs
    engine.use_graphs = False
    try:
        engine.step(entries, end=end)                          # warm
        totals: dict = {}
        seen = set()
        for _ in range(reps):
            # a long kernel ahead of the step lets the host queue every launch before the device starts on the
            # first: the sections then hold the kernels' own times, not the host's time between two launches
            torch.cuda._sleep(int(ahead_ms * 2.0e6))
            with SectionTimer() as t:
                logits = engine.step(entries, end=end)
                if logits is not None:
                    chosen = torch.zeros(logits.shape[0], dtype=torch.int32, device=logits.device)
                    ops.sample(logits, chosen)
            for what, note, ms in t.sections():
                c = classify(cfg, what, note)
                seen.add(what)
                n, total = totals.get(c, (0, 0.0))
                totals[c] = (n + 1, total + ms)
        out = Sections({c: (n / reps, total / reps) for c, (n, total) in totals.items()})
        out.ops = frozenset(seen)
        return out
    finally:
        engine.use_graphs = was


class TimelineUnavailable(RuntimeError):
    """The driver's activity records (CUPTI) cannot be had here: another profiler holds them, or the process may not."""


def decode_timeline(engine, batch: int, context: int, gen, warmup: int = 8) -> list:
    """The kernels of one decode step as the device ran them, from the driver's activity records (torch.profiler):
    [(start us, end us, name)] in order of start, times from the step's first kernel.  Unlike the section timer this
    leaves the step as it is (a replayed graph with programmatic dependent launches), so a kernel's start lies before
    the end of the one ahead of it; what a kernel costs the step is its end minus the end of the kernel before it."""
    from torch.profiler import ProfilerActivity, profile
    ids = seat(engine, [context] * batch)
    tok = torch.randint(0, engine.model.vocab_size, (batch,), generator=gen).tolist()
    entries = [Entry(r, [t], [0]) for r, t in zip(ids, tok)]
    chosen = torch.zeros(batch, dtype=torch.int32, device=engine.runtime.device)
    for _ in range(warmup):
        ops.sample(engine.step(entries), chosen, n=batch)
    torch.cuda.synchronize()
    try:
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                ops.sample(engine.step(entries), chosen, n=batch)
            torch.cuda.synchronize()
        events = list(prof.events())
    except RuntimeError as exc:                          # the profiler could not start
        engine.cache.release_all()
        raise TimelineUnavailable(str(exc)) from None
    rows = sorted(((e.time_range.start, e.time_range.end, e.name) for e in events
                   if "cuda" in str(e.device_type).lower() and "Memcpy" not in e.name and "Memset" not in e.name),
                  key=lambda r: r[0])
    firsts = [i for i, r in enumerate(rows) if "embedding" in r[2]]
    if len(firsts) < 3:
        engine.cache.release_all()
        raise TimelineUnavailable("the profiler returned no kernel records for the step")
    a, b = firsts[1], firsts[2]                          # the second of the three steps
    t0 = rows[a][0]
    engine.cache.release_all()
    return [(s - t0, e - t0, n) for s, e, n in rows[a:b]]


def attention_check(engine, batch: int, context: int, gen) -> dict:
    """Relative error of the bfloat16 decode attention over the cache of `batch` seated requests (layer call 0,
    a random query) against a float32 softmax over the same pages, for the first and the last sequence."""
    ids = seat(engine, [context] * batch)
    vocab = engine.model.vocab_size
    entries = [Entry(r, [int(torch.randint(0, vocab, (1,), generator=gen))], [0]) for r in ids]
    logits = engine.step(entries)                              # leaves the step's descriptor on the device
    finite = bool(torch.isfinite(logits).all())
    b = engine.last_batch
    mixer = engine.model.layers[engine.model.order[0].layer].mixer
    nh, nkv, hd, window, scale = mixer.nh, mixer.nkv, mixer.hd, mixer.window, mixer.scale
    view = engine.cache.view(0, b.tables, b.table_bases)
    dev = engine.runtime.device
    q = torch.randn(batch, nh * hd, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).to(view.k_pool.dtype)
    out = torch.empty_like(q)
    ops.paged_attention_mma(q, out, view.k_pool, view.v_pool, view.block_table, b.seq_q_start_d, b.seq_q_len_d,
                            b.seq_pos_start_d, batch, 1, context, True, False, nh, nkv, hd, window, scale,
                            engine.runtime.status, table_base=view.table_base)
    worst = 0.0
    page = engine.cache.page_size
    for s in sorted({0, batch - 1}):
        p = context - 1                                        # the query's position
        t0 = max(0, p - window + 1) if window else 0
        base = int(view.table_base[s]) if view.table_base is not None else 0
        row = view.block_table[s].long()
        pos = torch.arange(t0, p + 1, device=dev)
        pages = row[pos // page - base]
        k = view.k_pool[pages, :, pos % page].float()          # [keys, kv heads, hd]
        v = view.v_pool[pages, :, pos % page].float()
        qs = q[s].float().view(nkv, nh // nkv, hd)
        w = torch.softmax(scale * torch.einsum("kgd,tkd->kgt", qs, k), dim=-1)
        ref = torch.einsum("kgt,tkd->kgd", w, v).reshape(-1)
        worst = max(worst, float((out[s].float() - ref).abs().max() / ref.abs().max()))
    engine.runtime.check_status("attention check")
    for rid in ids:
        engine.cache.release(rid)
    return {"decode_attention_rel_err": round(worst, 5), "logits_finite": finite, "sequences": batch,
            "context": context}


def mixed_requests(engine, *, n_requests: int, prompt_range: tuple, chunk: int, ubatch: int, decode_tokens: int,
                   temperature: float, seed: int) -> dict:
    """`n_requests` requests with seeded prompt lengths, all handed over at time 0, through the scheduler's loop.
    Times are taken on the host when a token has arrived there."""
    rng = random.Random(seed)
    lengths = [rng.randint(*prompt_range) for _ in range(n_requests)]
    vocab = engine.model.vocab_size
    prompts = [[rng.randrange(vocab) for _ in range(n)] for n in lengths]
    engine.cache.release_all()
    ex = EngineExecutor(engine)
    sched = Scheduler(ex, token_budget=ubatch, prefill_chunk=chunk, max_running=engine.options.max_requests)
    reqs = [sched.add(i, p, SamplingParams(temperature=temperature, seed=seed + i, max_tokens=decode_tokens,
                                           ignore_eos=True)) for i, p in enumerate(prompts)]
    first, last, step_rows = {}, {}, []
    trace = os.environ.get("FLAMBEAU_BENCH_TRACE")          # one line per step on stderr
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while not sched.idle:
        out = sched.step()
        now = time.perf_counter() - t0
        if trace:
            b = engine.last_batch
            print(f"[mixed {now:8.3f} s] step {sched.steps}: {b.n_tokens} rows of {b.n_seqs} sequences, "
                  f"{len(out)} tokens out, {len(sched.running)} running, {len(sched.waiting)} waiting",
                  file=sys.stderr, flush=True)
        for r, _tok in out:
            first.setdefault(r.request_id, now)
            last[r.request_id] = now
        if engine.last_batch is not None:
            step_rows.append(engine.last_batch.n_tokens)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    engine.runtime.check_status("mixed workload")
    engine.cache.check_invariants()
    generated = sum(len(r.generated) for r in reqs)
    ttft = [first[r.request_id] for r in reqs]
    prefill_rates = [len(r.prompt) / first[r.request_id] for r in reqs]
    decode_rates = [(len(r.generated) - 1) / (last[r.request_id] - first[r.request_id]) for r in reqs
                    if len(r.generated) > 1 and last[r.request_id] > first[r.request_id]]
    return {
        "requests": n_requests, "prompt_tokens": sum(lengths), "generated_tokens": generated, "wall_s": round(wall, 3),
        "tokens_per_s": round((sum(lengths) + generated) / wall, 1),
        "generated_per_s": round(generated / wall, 1),
        "prefill_tok_s_median": round(statistics.median(prefill_rates), 1),
        "prefill_tok_s_aggregate": round(sum(lengths) / max(ttft), 1),
        "ttft_ms_median": round(statistics.median(ttft) * 1e3, 1), "ttft_ms_max": round(max(ttft) * 1e3, 1),
        "decode_tok_s_median": round(statistics.median(decode_rates), 2) if decode_rates else None,
        "steps": sched.steps, "steps_ahead": sched.steps_ahead, "rows_per_step_mean": round(statistics.mean(step_rows), 1),
        "preemptions": sum(r.preemptions for r in reqs),
        "finish": sorted({r.finish_reason for r in reqs}),
    }


def step_host_device(engine, *, decoding: int, context: int, portion: int, gen, reps: int = 4) -> dict:
    """One mixed step (a prompt portion of `portion` tokens beside `decoding` decoded tokens at `context`): the
    host's time to plan nothing, pack and launch it; the device's time for it when every launch is already
    queued (a long kernel ahead of the step lets the host run ahead); and the time a caller sees with nothing to
    hide the host behind."""
    vocab = engine.model.vocab_size

    def entries():
        ids = seat(engine, [context] * decoding + [portion + 1], prefix="m")
        e = [Entry(r, [int(torch.randint(0, vocab, (1,), generator=gen))], [0]) for r in ids[:-1]]
        e.append(Entry(ids[-1], torch.randint(0, vocab, (portion,), generator=gen).tolist(), []))
        return e

    engine.step(entries())                                     # warm
    torch.cuda.synchronize()
    host, device, seen = [], [], []
    for _ in range(reps):
        batch = entries()
        torch.cuda._sleep(60_000_000)                          # ~30 ms of device time for the host to run ahead of
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        w0 = time.perf_counter()
        engine.step(batch)
        host.append((time.perf_counter() - w0) * 1e3)
        e1.record()
        torch.cuda.synchronize()
        device.append(e0.elapsed_time(e1))
        batch = entries()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        engine.step(batch)
        torch.cuda.synchronize()
        seen.append((time.perf_counter() - w0) * 1e3)
    engine.runtime.check_status("mixed step")
    engine.cache.release_all()
    h, d, s = statistics.median(host), statistics.median(device), statistics.median(seen)
    return {"rows": portion + decoding, "host_ms": round(h, 3), "device_ms": round(d, 3), "alone_ms": round(s, 3),
            "host_share_alone": round(max(0.0, s - d) / s, 3)}


def roofline_of_sections(cfg, sections: dict, rows: int, contexts, layers: int, peaks: dict) -> dict:
    """Fold measured sections into the bench line's `kernels` object: per class, launches and microseconds per
    layer call (per step for the head and the sampler), the work, and the fraction of the measured peak that
    bounds it (memory for few rows and for the row-wise kernels, the tensor cores for products and attention over
    hundreds of rows)."""
    # (whether the projections added to the residual stream themselves is what the step did, where that is known)
    ops_seen = getattr(sections, "ops", None)
    classes = work.kernel_classes(cfg, rows, contexts, to_stream=None if ops_seen is None else "gemm_tc_add" in ops_seen)
    out = {}
    for name, (launches, ms) in sections.items():
        per = 1 if name in ("lm_head", "sample", "embedding", "rope_table") else layers
        if name == "add_norm":
            per = 2 * layers + 1                               # two a layer and the final one
            launches_per, us = launches / per, ms * 1e3 / per
        else:
            launches_per, us = launches / per, ms * 1e3 / per
        rec = {"launches": round(launches_per, 2), "us": round(us, 2)}
        w = classes.get(name)
        if w and us > 0:
            gbs = w["bytes"] / (us * 1e-6) / 1e9
            tflops = w["flops"] / (us * 1e-6) / 1e12
            by_mem = gbs / peaks["hbm_gbs"]
            by_math = tflops / peaks["bf16_tflops"]
            if by_math > by_mem:
                rec.update(bound="tensor", achieved=round(tflops, 1), unit="TFLOP/s", frac=round(by_math, 3))
            else:
                rec.update(bound="hbm", achieved=round(gbs, 1), unit="GB/s", frac=round(by_mem, 3))
        out[name] = rec
    return out
