#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of the Mistral-7B-v0.1 shape with random weights in bfloat16, a batch of 8
sequences that each hold 8,192 tokens of context (4,096 live keys under the sliding window), 16-token pages.
A "step" is one decode step.  It prints ONE JSON line:

  value      decoded tokens a second, timed on the device with CUDA events over exactly K steps
  e2e        the same through the Python entry point's own loop (scheduler step -> engine step -> sampler):
             host token ids in from pinned memory, sampled token ids back to the host, every step
  prefill    one step of 2,048 prompt tokens: tokens a second, ms, and flops / time / bf16 peak
  roofline   bytes the decode step has to read (every weight it uses once + the live cache) / time / HBM peak
  points     decode tokens a second at batch 1 and 64

The cache of the timed sequences is laid out by the cache manager exactly as a real 8,192-token request leaves
it (pages taken and, under the window, given back), but its keys and values are random numbers rather than the
result of 8 x 8,192 tokens of prefill; weights are random too ("data": "synthetic").
Every decode step reads all weights (14 GB), far more than the 126 MB L2, so no L2 flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

MISTRAL_7B = dict(architectures=["MistralForCausalLM"], hidden_size=4096, num_hidden_layers=32,
                  num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
                  vocab_size=32000, rope_theta=10000.0, sliding_window=4096, rms_norm_eps=1e-5,
                  tie_word_embeddings=False, max_position_embeddings=32768)


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            raw = json.loads(p.read_text())
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)) and k not in flat:
                        flat[k] = float(v)
            walk(raw)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return {"hbm_gbs": flat["hbm_gbs"], "bf16_tflops": flat["bf16_tflops"],
                        "bf16_tflops_sustained": flat.get("bf16_tflops_sustained"), "source": "measured"}
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the 32 of the shape (sizes unchanged)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--skip-points", action="store_true", help="do not measure batch 1 and 64")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "arte-fact/flambeau is a Rust workspace with HIP kernels for AMD gfx906: it has no Python "
                          "package to install (pip finds no setup.py or pyproject.toml), no cargo or hipcc here, and "
                          "no CUDA path or Mistral model to run on a B200"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from flambeau_b200.config.mistral import MistralConfig
    from flambeau_b200.engine.batch import Entry
    from flambeau_b200.engine.generate import EngineExecutor
    from flambeau_b200.engine.scheduler import Request, Scheduler
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.kernels import library
    from flambeau_b200.sampling.params import SamplingParams

    pk = peaks()
    layers_full = MISTRAL_7B["num_hidden_layers"]
    layers = args.layers or layers_full
    cfg = MistralConfig.from_dict({**MISTRAL_7B, "num_hidden_layers": layers})
    window = cfg.sliding_window or 0
    page = 16
    max_batch = args.batch if args.skip_points else max(args.batch, 64)
    live_per_seq = min(args.context, window + page) if window else args.context
    per_seq_pool = -(-(live_per_seq + 2 * page + args.steps + args.warmup + 64) // page) * page
    cache_tokens = max(max_batch * per_seq_pool + 512, args.prefill_tokens + page)
    engine = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype="bfloat16", page_size=page, cache_tokens=cache_tokens, max_requests=max_batch,
        max_step_tokens=max(args.prefill_tokens, max_batch), max_seq_len=args.context + 4096))
    dev = engine.runtime.device
    for g in engine.cache.groups:                       # random keys and values stand in for a real prefill
        for c in g.owners:
            g.k[c].normal_(0.0, 1.0)
            g.v[c].normal_(0.0, 1.0)
    vocab = cfg.vocab_size
    gen = torch.Generator().manual_seed(1)

    def seat(batch: int, context: int) -> list:
        """`batch` requests whose cache holds context-1 tokens (bookkeeping only: pages taken and released as a
        real request of that length would have them)."""
        engine.cache.release_all()
        ids = []
        for i in range(batch):
            rid = f"seq{i}"
            engine.cache.admit(rid)
            left = context - 1
            while left > 0:
                k = min(left, 256)
                engine.cache.reserve(rid, k)
                engine.cache.commit(rid, k)
                left -= k
            ids.append(rid)
        return ids

    def decode_device(batch: int, steps: int, warmup: int) -> tuple:
        """(ms per step, launches per step) of engine.step + on-device sampling with fixed input tokens."""
        ids = seat(batch, args.context)
        tok = torch.randint(0, vocab, (batch,), generator=gen).tolist()
        entries = [Entry(r, [t], [0]) for r, t in zip(ids, tok)]
        from flambeau_b200.kernels import ops
        chosen = torch.zeros(batch, dtype=torch.int32, device=dev)
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
        engine.runtime.check_status("bench decode")
        return t0.elapsed_time(t1) / steps, (library.LAUNCHES[0] - l0) / steps

    def decode_e2e(batch: int, steps: int, warmup: int) -> tuple:
        """Tokens a second through the scheduler loop that generate() runs: host ids in, host ids out."""
        ids = seat(batch, args.context)
        ex = EngineExecutor(engine)
        sched = Scheduler(ex, token_budget=max(batch, 1), prefill_chunk=512, max_running=batch)
        for i, rid in enumerate(ids):
            r = Request(rid, prompt=[0] * (args.context - 1), params=SamplingParams(max_tokens=steps + warmup + 8),
                        generated=[int(torch.randint(0, vocab, (1,), generator=gen))], arrival=i)
            r.fed = args.context - 1
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

    def prefill(tokens: int) -> float:
        engine.cache.release_all()
        toks = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
        times = []
        for i in range(8):                              # 3 warm-up steps, then the median of 5
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            engine.step([Entry("prompt", toks, [tokens - 1])], end=["prompt"])
            t1.record()
            torch.cuda.synchronize()
            if i >= 3:
                times.append(t0.elapsed_time(t1))
        engine.runtime.check_status("bench prefill")
        return statistics.median(times)

    # ---- measurements ----------------------------------------------------------
    with ClockSampler(dev.index or 0) as clocks:        # clocks and throttle reasons while the timed regions run
        time.sleep(0.3)                                 # let nvidia-smi start reporting before the first region
        ms_step, launches = decode_device(args.batch, args.steps, args.warmup)
        e2e_value, h2d, d2h = decode_e2e(args.batch, args.steps, args.warmup)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                ms_b, _ = decode_device(b, max(8, args.steps // 2), 3)
                points[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)
        pre_ms = prefill(args.prefill_tokens)
    clock_summary = clocks.summary()

    # ---- accounting --------------------------------------------------------------
    weight_bytes = engine.model.step_weight_bytes()
    live_keys = min(args.context, window) if window else args.context
    kv_bytes = args.batch * live_keys * engine.cache.kv_bytes_per_token()
    step_bytes = weight_bytes + kv_bytes
    achieved_gbs = step_bytes / (ms_step / 1e3) / 1e9
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qw, kvw = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    T = args.prefill_tokens
    linear_flops = 2.0 * T * layers * (H * (qw + 2 * kvw) + qw * H + 3 * H * I) + 2.0 * V * H
    # causal attention within the window: query i sees min(i+1, W) keys; QK^T and PV, 2 flops per multiply-add
    seen = sum(min(i + 1, window) if window else i + 1 for i in range(T))
    attn_flops = 2.0 * 2.0 * seen * qw * layers
    pre_flops = linear_flops + attn_flops
    pre_tflops = pre_flops / (pre_ms / 1e3) / 1e12
    value = args.batch / (ms_step / 1e3)
    tag = "of measured" if pk["source"] == "measured" else "of fallback"
    line = {
        "metric": "decode tok/s @ batch 8 (Mistral-7B shape, 8192 context); prefill tok/s @ 2048; % of roofline",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "Mistral-7B-v0.1 shape, random weights", "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single GPU", "layers": layers, "layers_of_shape": layers_full, "hidden_size": H,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate_size": I, "vocab_size": V, "sliding_window": window, "page_size": page,
            "kv_dtype": "bf16", "l2": "inputs larger than L2 (every step reads all weights)",
            "cache_state": "pages laid out by the cache manager for 8191-token requests; K/V values random",
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(pre_tflops / pk["bf16_tflops"], 4), "tflops": round(pre_tflops, 1),
                    "peak_tflops": pk["bf16_tflops"], "peak": tag},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes),
                     "peak_source": tag},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
