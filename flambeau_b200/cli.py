"""Command line in the manner of the reference's `flambeau` binary
(crates/cli/src/main.rs:36-278): subcommands, long options with dashes.

  flambeau infer --model DIR --prompt "1,2,3" --max-tokens 64 [--temperature T --top-p P --top-k K --min-p M
                 --seed S --dtype bfloat16|float32 --devices cuda:0 --inflight-slots N --prefill-ubatch N
                 --prefill-chunk-tokens N --paged-kv PAGES --ctx-cap N]
  flambeau replay --model DIR --dtype ... --out DIR --max-tokens N      (steps as JSON lines on stdin)
  flambeau random-model --config CONFIG.json --out DIR --seed S --dtype bfloat16|float32
  flambeau inspect --model DIR
  flambeau bench [--shape 7b|nemo12b|small24b] [--only headline|mixed|shapes] [--steps K] ...   (one JSON line)

The reference's `infer` takes text and a tokenizer from its model file; this engine takes token ids, so
`--prompt` is a list of ids (commas or spaces) and the completion is printed as ids.
"""
from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str) -> list:
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_infer(a) -> int:
    from .engine.generate import generate
    prompts = [_ids(p) for p in a.prompt]
    if a.prompt_file:
        for line in open(a.prompt_file):
            if line.strip():
                prompts.append(_ids(line))
    if not prompts:
        print("infer: no prompt given (--prompt or --prompt-file)", file=sys.stderr)
        return 2
    outs = generate(a.model, prompts, max_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p,
                    top_k=a.top_k, min_p=a.min_p, repetition_penalty=a.repetition_penalty,
                    presence_penalty=a.presence_penalty, frequency_penalty=a.frequency_penalty, seed=a.seed,
                    stop_token_ids=tuple(a.stop_token_id or ()), dtype=a.dtype, devices=a.devices,
                    inflight_slots=a.inflight_slots, prefill_ubatch=a.prefill_ubatch,
                    prefill_chunk_tokens=a.prefill_chunk_tokens, paged_kv=a.paged_kv, ctx_cap=a.ctx_cap)
    for o in outs:
        print(",".join(str(t) for t in o))
    return 0


def cmd_replay(a) -> int:
    from .engine.trace import main as trace_main
    return trace_main(["--model", a.model, "--dtype", a.dtype, "--out", a.out, "--max-tokens", str(a.max_tokens)])


def cmd_random_model(a) -> int:
    from . import models  # noqa: F401
    from .config.base import ConfigReader, read_config_json
    from .config.registry import resolve
    from .weights.random_init import write_random_model
    raw = read_config_json(a.config)
    cfg = resolve(ConfigReader(raw).architecture()).config_class.from_dict(raw)
    write_random_model(a.out, cfg, seed=a.seed, dtype=a.dtype)
    print(a.out)
    return 0


def cmd_inspect(a) -> int:
    from . import models  # noqa: F401
    from .config.registry import load_config
    from .weights.safetensors_io import ModelFiles
    arch, cfg = load_config(a.model)
    print(json.dumps({"architecture": arch.name, "config": cfg.to_dict()}, indent=2))
    files = ModelFiles(a.model)
    for name in sorted(files.names()):
        print(f"{name}\t{files.dtype(name)}\t{list(files.shape(name))}")
    return 0


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else list(argv)
    if argv and argv[0] == "bench":                # the benchmark parses its own options
        from .measure.bench import main as bench_main
        return bench_main(argv[1:])
    ap = argparse.ArgumentParser(prog="flambeau", description="B200-native single-GPU inference engine")
    sub = ap.add_subparsers(dest="cmd", required=True)

    p = sub.add_parser("infer", help="generate from prompts given as token ids")
    p.add_argument("--model", required=True)
    p.add_argument("--prompt", action="append", default=[], help='token ids, e.g. "1,2,3"; may be repeated')
    p.add_argument("--prompt-file", help="one prompt per line")
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("--devices", default="cuda:0")
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-p", type=float)
    p.add_argument("--top-k", type=int)
    p.add_argument("--min-p", type=float)
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--presence-penalty", type=float, default=0.0)
    p.add_argument("--frequency-penalty", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--stop-token-id", type=int, action="append")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--inflight-slots", type=int, default=4)
    p.add_argument("--prefill-ubatch", type=int, default=2048, help="most rows of one step")
    p.add_argument("--prefill-chunk-tokens", type=int, default=2048, help="longest portion of a prompt in one step")
    p.add_argument("--paged-kv", type=int, help="number of cache pages (16 tokens each)")
    p.add_argument("--ctx-cap", type=int)
    p.set_defaults(fn=cmd_infer)

    p = sub.add_parser("replay", help="feed given token ids step by step and write logits")
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, required=True)
    p.set_defaults(fn=cmd_replay)

    p = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    p.add_argument("--config", required=True, help="a config.json (file or folder)")
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.set_defaults(fn=cmd_random_model)

    p = sub.add_parser("inspect", help="print the configuration and the tensor list of a model folder")
    p.add_argument("--model", required=True)
    p.set_defaults(fn=cmd_inspect)

    sub.add_parser("bench", help="decode and prefill throughput with rooflines, as one JSON line "
                                 "(`flambeau bench --help` lists its options)")

    a = ap.parse_args(argv)
    from .errors import USER_ERRORS
    try:
        return a.fn(a)
    except USER_ERRORS as e:                       # what the input can cause: one line, no trace
        sys.stderr.write(f"flambeau {a.cmd}: error: {type(e).__name__}: {e}\n")
        return 1


if __name__ == "__main__":
    sys.exit(main())
