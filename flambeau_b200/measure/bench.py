"""Decode and prefill throughput of the engine on one B200.

    python bench.py | flambeau bench  [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                                      [--shape 7b|nemo12b|small24b] [--only headline|mixed|shapes] ...

Default run: the layer sizes of the Mistral-7B-v0.1 shape with random weights in bfloat16, a batch of 8
sequences that each hold 8,192 tokens of context (4,096 live keys under the sliding window), 16-token pages.
A "step" is one decode step.  It prints ONE JSON line:

  value      decoded tokens a second, timed on the device with CUDA events over exactly K steps
  e2e        the same through the Python entry point's own loop (scheduler step -> engine step -> sampler):
             host token ids in from pinned memory, sampled token ids back to the host, every step
  prefill    one step of 2,048 prompt tokens: tokens a second, ms, and flops / time / bf16 peak; beside it the
             same prompt through the entry point as time to the first token (`ttft_ms`, the scheduler cutting it
             into portions of 512, the default, and of 2,048) and one bare step of 512 tokens
  roofline   bytes the decode step has to read (every weight it uses once + the live cache) / time / HBM peak
  points     decode tokens a second at batch 1 and 64, and the other shapes' figures as flat numbers
  kernels    per kernel class of the decode step and of the 2,048-token step: launches and microseconds per layer
             call (CUDA events around every launcher call of an eager step: serialised kernels), and the
             fraction of the measured peak that bounds the class
  check      outside the timed regions: the decode attention at the benchmarked geometry against a float32
             softmax over the same pages, and whether the step's logits are finite
  mixed      the Mistral-Nemo-12B shape: 32 requests with seeded prompts of 128 to 4,096 tokens, portions of
             512, 256 sampled tokens each at temperature 0.7, through the scheduler with a page pool smaller
             than the requests' sum; prefill as prompt tokens / time to first token and decode as
             (n - 1) / (last - first token time), the reference's conventions (doc/PERF_MATRIX.md:4-8); and one
             mixed step's host time against its device time
  shapes     the Mistral-Small-24B shape: decode at batch 1 / 8 / 64 with 4,096-token contexts and a 2,048-token
             prefill, each with its roofline fraction

The cache of the timed sequences is laid out by the cache manager exactly as a real request of that length
leaves it (pages taken and, under the window, given back), but its keys and values are random numbers rather than
the result of a prefill; weights are random too ("data": "synthetic").  Every decode step reads all weights
(14 GB and more), far more than the 126 MB L2, so no L2 flush is needed.
"""
from __future__ import annotations

import argparse
import gc
import json
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]          # MEASURED_PEAKS.json lies beside the package

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
PAGE = 16


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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--shape", default="7b", help="the shape of the headline run: 7b, nemo12b or small24b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None, help="tokens per sequence (default: the shape's)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (sizes unchanged)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--skip-points", action="store_true", help="do not measure batch 1 and 64")
    ap.add_argument("--only", choices=["all", "headline", "mixed", "shapes", "timeline", "mma-issue"], default="all",
                    help="headline: the shape's own line only; mixed / shapes: that part only; timeline: the kernels "
                         "of one decode step at --batch as the device ran them (a table on stderr, 4 layers unless "
                         "--layers says otherwise); mma-issue: cycles per tcgen05.mma of one SM for the attention "
                         "kernel's instruction streams (a table on stderr)")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "arte-fact/flambeau is a Rust workspace with HIP kernels for AMD gfx906: it has no Python "
                          "package to install (pip finds no setup.py or pyproject.toml), no cargo or hipcc here, and "
                          "no CUDA path or Mistral model to run on a B200"}))
        return 0
    if args.gpus != 1:
        print(f"bench: this engine runs on one GPU; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import os
    if os.environ.get("FLAMBEAU_BENCH_STACKS"):          # where the host is after that many seconds (diagnosis)
        import faulthandler
        faulthandler.dump_traceback_later(float(os.environ["FLAMBEAU_BENCH_STACKS"]), repeat=False, file=sys.stderr)
    import torch
    from flambeau_b200.config.mistral import MistralConfig
    from flambeau_b200.engine.batch import Entry
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.measure import work, workloads
    from flambeau_b200.measure.shapes import shape as shape_of
    from flambeau_b200.measure.timers import ClockSampler

    pk = peaks()
    tag = "of measured" if pk["source"] == "measured" else "of fallback"
    gen = torch.Generator().manual_seed(1)
    started = time.time()

    def say(msg: str) -> None:                           # progress on stderr; stdout carries the JSON line alone
        print(f"[bench {time.time() - started:6.1f} s] {msg}", file=sys.stderr, flush=True)

    def build(shape, layers, max_batch, context, prefill_tokens, steps):
        cfg = MistralConfig.from_dict({**shape.config, "num_hidden_layers": layers})
        window = cfg.sliding_window or 0
        live = min(context, window + PAGE) if window else context
        per_seq = -(-(live + 2 * PAGE + steps + 64) // PAGE) * PAGE
        cache_tokens = max(max_batch * per_seq + 512, prefill_tokens + PAGE)
        engine = Engine.from_config(cfg, seed=0, options=EngineOptions(
            dtype="bfloat16", page_size=PAGE, cache_tokens=cache_tokens, max_requests=max_batch,
            max_step_tokens=max(prefill_tokens, max_batch), max_seq_len=min(context + 4096, cfg.max_position_embeddings)))
        workloads.randomise_cache(engine)
        return cfg, engine

    def free_device_memory():
        gc.collect()
        torch.cuda.empty_cache()

    def decode_point(engine, cfg, batch, context, steps, warmup):
        ms, launches = workloads.decode_device(engine, batch, context, steps, warmup, gen)
        nbytes = work.decode_step_bytes(engine.model.step_weight_bytes(), engine.cache.kv_bytes_per_token(),
                                        [context] * batch, cfg.sliding_window or 0)
        gbs = nbytes / (ms / 1e3) / 1e9
        return dict(ms=ms, launches=launches, tok_s=batch / (ms / 1e3), bytes=nbytes, gbs=gbs,
                    frac=gbs / pk["hbm_gbs"])

    def prefill_point(engine, cfg, layers, tokens):
        ms = workloads.prefill_step(engine, tokens, gen)
        flops = work.step_flops(cfg, layers, range(tokens), 1)
        tflops = flops / (ms / 1e3) / 1e12
        return dict(ms=ms, tok_s=tokens / (ms / 1e3), tflops=tflops, frac=tflops / pk["bf16_tflops"])

    line: dict = {}
    clock_summary = None
    head = shape_of(args.shape)
    context = args.context or head.context
    layers_full = head.config["num_hidden_layers"]
    layers = args.layers or layers_full

    if args.only == "mma-issue":
        from flambeau_b200.measure.probes import run_probe
        table = run_probe("mma_issue_rate")
        print(table, file=sys.stderr)
        rows = [ln.rsplit(None, 4) for ln in table.splitlines()[1:] if ln.strip()]
        print(json.dumps({"impl": "ours", "mma_issue_cycles_each": {r[0].strip(): float(r[3]) for r in rows}}))
        return 0
    if args.only == "timeline":
        layers = args.layers or 4
        say(f"building {head.name}, {layers} layers")
        cfg, engine = build(head, layers, args.batch, context, args.batch, 64)
        rows = workloads.decode_timeline(engine, args.batch, context, gen)
        last_end, costs = 0.0, {}
        print(f"{'start us':>9} {'end us':>9} {'alone us':>9} {'costs us':>9}  kernel", file=sys.stderr)
        for start, end, name in rows:
            short = name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
            cost = max(end - last_end, 0.0)
            print(f"{start:9.2f} {end:9.2f} {end - start:9.2f} {cost:9.2f}  {short}", file=sys.stderr)
            costs[short] = costs.get(short, 0.0) + cost
            last_end = max(last_end, end)
        print(json.dumps({"impl": "ours", "timeline": {"model": head.name, "layers": layers, "batch": args.batch,
                          "context": context, "step_us": round(last_end, 2),
                          "cost_us_by_kernel": {k: round(v, 2) for k, v in costs.items()}}}))
        return 0

    with ClockSampler(0) as clocks:                     # clocks and throttle reasons while the timed regions run
        time.sleep(0.3)                                 # let nvidia-smi start reporting before the first region
        # ---- the headline shape -------------------------------------------------------------------
        if args.only in ("all", "headline"):
            max_batch = args.batch if args.skip_points else max(args.batch, 64)
            say(f"building {head.name}, {layers} layers")
            cfg, engine = build(head, layers, max_batch, context, args.prefill_tokens, args.steps + args.warmup)
            say(f"decode at batch {args.batch}")
            d = decode_point(engine, cfg, args.batch, context, args.steps, args.warmup)
            say(f"{d['ms']:.3f} ms a step; the same through the scheduler loop")
            e2e_value, h2d, d2h = workloads.decode_e2e(engine, args.batch, context, args.steps, args.warmup, gen)
            points = {}
            if not args.skip_points:
                for b in (1, 64):
                    points[f"decode_b{b}"] = round(decode_point(engine, cfg, b, context, max(8, args.steps // 2), 3)["tok_s"], 1)
            T = args.prefill_tokens
            say(f"prefill of {T} tokens")
            pre = prefill_point(engine, cfg, layers, T)
            prefill = {"value": round(pre["tok_s"], 1), "tokens": T, "ms": round(pre["ms"], 3),
                       "frac": round(pre["frac"], 4), "tflops": round(pre["tflops"], 1),
                       "peak_tflops": pk["bf16_tflops"], "peak": tag}
            if pk.get("bf16_tflops_sustained"):
                # the library product's figure from a seconds-long loop under the power cap, beside the burst figure
                # that `frac` is of: the timed steps follow each other, so the board is at its cap here too
                prefill["frac_of_sustained"] = round(pre["tflops"] / pk["bf16_tflops_sustained"], 4)
            if args.only == "all":
                pre512 = prefill_point(engine, cfg, layers, 512)
                prefill["step_512_ms"] = round(pre512["ms"], 3)
                prefill["step_512_tok_s"] = round(pre512["tok_s"], 1)
                for chunk in (512, T):
                    say(f"time to first token, portions of {chunk}")
                    ms = workloads.time_to_first(engine, T, chunk, gen)
                    prefill[f"ttft_ms_chunk{chunk}"] = round(ms, 3)
                    prefill[f"ttft_tok_s_chunk{chunk}"] = round(T / (ms / 1e3), 1)
            # ---- outside the timed regions: correctness of the benchmarked geometry, per-kernel times ----
            say("attention check and kernel sections")
            check = workloads.attention_check(engine, args.batch, context, gen)
            kernels = {}
            if args.only == "all":
                ids = workloads.seat(engine, [context] * args.batch)
                entries = [Entry(r, [int(torch.randint(0, cfg.vocab_size, (1,), generator=gen))], [0]) for r in ids]
                sections = workloads.kernel_sections(engine, entries, cfg)
                kernels[f"decode_b{args.batch}"] = workloads.roofline_of_sections(
                    cfg, sections, args.batch, [context] * args.batch, layers, pk)
                engine.cache.release_all()
                toks = torch.randint(0, cfg.vocab_size, (T,), generator=gen).tolist()
                for rows in (T, 512):
                    sections = workloads.kernel_sections(engine, [Entry("prompt", toks[:rows], [rows - 1])], cfg,
                                                         end=["prompt"])
                    kernels[f"prefill_{rows}"] = workloads.roofline_of_sections(cfg, sections, rows, [rows], layers, pk)
            window = cfg.sliding_window or 0
            line = {
                "metric": f"decode tok/s @ batch {args.batch} ({head.name}, {context} context); "
                          f"prefill tok/s @ {T}; % of roofline",
                "value": round(d["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(d["ms"], 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
                "config": {
                    "model": f"{head.name}, random weights", "global_batch": args.batch, "seq_len": context,
                    "parallelism": "single GPU", "layers": layers, "layers_of_shape": layers_full,
                    "hidden_size": cfg.hidden_size, "heads": cfg.num_attention_heads,
                    "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                    "intermediate_size": cfg.intermediate_size, "vocab_size": cfg.vocab_size,
                    "sliding_window": window, "page_size": PAGE, "kv_dtype": "bf16",
                    "l2": "inputs larger than L2 (every step reads all weights)",
                    "cache_state": f"pages laid out by the cache manager for {context - 1}-token requests; K/V values random",
                },
                "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                        "d2h_bytes_per_step": int(d2h)},
                "gpu_launches": int(round(d["launches"] * args.steps)),
                "prefill": prefill,
                "roofline": {"bound": "hbm", "achieved": round(d["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": round(d["frac"], 4), "bytes_per_step": int(d["bytes"]), "peak_source": tag},
                "points": points, "check": check, "kernels": kernels,
            }
            engine = None
            free_device_memory()

        # ---- the Mistral-Nemo-12B mixed workload through the scheduler -----------------------------------
        if args.only in ("all", "mixed"):
            nemo = shape_of("nemo12b")
            ncfg = MistralConfig.from_dict(nemo.config if args.layers is None else
                                           {**nemo.config, "num_hidden_layers": args.layers})
            n_req, lo, hi, chunk, new = 32, 128, 4096, 512, 256
            ubatch = 2 * chunk + n_req                        # two portions beside every decoded token
            demand = n_req * ((lo + hi) // 2 + new)           # about what the requests come to hold together
            say(f"building {nemo.name}, {ncfg.num_hidden_layers} layers")
            engine = Engine.from_config(ncfg, seed=0, options=EngineOptions(
                dtype="bfloat16", page_size=PAGE, cache_tokens=int(0.75 * demand) // PAGE * PAGE, max_requests=n_req,
                max_step_tokens=ubatch, max_seq_len=hi + new + PAGE))
            say("mixed workload: warm-up")
            workloads.mixed_requests(engine, n_requests=4, prompt_range=(lo, 600), chunk=chunk, ubatch=ubatch,
                                     decode_tokens=8, temperature=0.7, seed=99)        # warm-up
            say(f"mixed workload: {n_req} requests")
            mixed = workloads.mixed_requests(engine, n_requests=n_req, prompt_range=(lo, hi), chunk=chunk,
                                             ubatch=ubatch, decode_tokens=new, temperature=0.7, seed=7)
            mixed.update(model=nemo.name, layers=ncfg.num_hidden_layers, layers_of_shape=nemo.config["num_hidden_layers"],
                         chunk=chunk, ubatch=ubatch, temperature=0.7, pool_tokens=engine.options.cache_tokens)
            say(f"{mixed['wall_s']} s; one mixed step, host against device")
            workloads.randomise_cache(engine)
            mixed["one_step"] = workloads.step_host_device(engine, decoding=24, context=2048, portion=chunk, gen=gen)
            line["mixed"] = mixed
            engine = None
            free_device_memory()

        # ---- the Mistral-Small-24B shape ------------------------------------------------------------------
        if args.only in ("all", "shapes"):
            big = shape_of("small24b")
            blayers = args.layers or big.config["num_hidden_layers"]
            say(f"building {big.name}, {blayers} layers")
            bcfg, engine = build(big, blayers, 64, big.context, 2048, args.steps + args.warmup)
            rec = {"model": big.name, "layers": blayers, "layers_of_shape": big.config["num_hidden_layers"],
                   "context": big.context, "peak": tag}
            for b in (1, 8, 64):
                say(f"decode at batch {b}")
                d = decode_point(engine, bcfg, b, big.context, max(8, args.steps // 2), 3)
                rec[f"decode_b{b}"] = {"value": round(d["tok_s"], 1), "ms": round(d["ms"], 3),
                                       "gbs": round(d["gbs"], 1), "frac": round(d["frac"], 4)}
                line.setdefault("points", {})[f"small24b_decode_b{b}"] = round(d["tok_s"], 1)
            pre = prefill_point(engine, bcfg, blayers, 2048)
            rec["prefill_2048"] = {"value": round(pre["tok_s"], 1), "ms": round(pre["ms"], 3),
                                   "tflops": round(pre["tflops"], 1), "frac": round(pre["frac"], 4)}
            ms = workloads.time_to_first(engine, 2048, 512, gen)
            rec["prefill_2048"]["ttft_ms_chunk512"] = round(ms, 3)
            line.setdefault("points", {})["small24b_prefill_2048"] = round(pre["tok_s"], 1)
            line["shapes"] = {"small24b": rec}
            engine = None
            free_device_memory()
    say("done")
    clock_summary = clocks.summary()
    line["clocks"] = clock_summary
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
