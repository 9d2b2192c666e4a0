"""Trace replay: feed given token ids through the engine step by step and write
the logits at the wanted places.  It samples nothing and has no forward pass,
cache or loader of its own: it drives Engine.step, the same call that
generation makes.

The reference's analogue feeds a fixed token list one token per step and dumps
`[len][len x f32]` records that a script diffs across builds
(crates/models/qwen35-v2/tests/parity_dump_v2.rs:14-61,
scripts/parity/v2_vs_legacy.sh:31-62); it does not replay schedules.

Input: one JSON object a line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: `<out>/<step>.f32`, little-endian float32 [wanted, vocab], for every
step that wants something; after every step a line `done <step>` on stdout.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

from .batch import Entry
from .step import Engine, EngineOptions


class TraceError(ValueError):
    pass


def replay(engine: Engine, lines, out_dir, report=None) -> int:
    """Run every step in `lines` (an iterable of JSON strings); returns the number of steps run."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    count = 0
    for raw in lines:
        raw = raw.strip()
        if not raw:
            continue
        try:
            rec = json.loads(raw)
            step = rec["step"]
            entries = [Entry(e["id"], list(e["tokens"]), list(e.get("want", []))) for e in rec.get("entries", [])]
        except (ValueError, KeyError, TypeError) as e:
            raise TraceError(f"input line {count + 1} is not a step record: {type(e).__name__}: {e}") from None
        logits = engine.step(entries, end=rec.get("end", []))
        if logits is not None and logits.shape[0] > 0:
            host = logits.float().cpu().contiguous().numpy().astype("<f4", copy=False)
            host.tofile(out_dir / f"{step}.f32")
        engine.runtime.check_status(f"step {step}")
        count += 1
        if report is not None:
            report(step)
    return count


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-requests", type=int, default=8)
    args = ap.parse_args(argv)
    tokens = max(64, -(-args.max_tokens // 64) * 64)

    def report(step):
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()

    from ..errors import USER_ERRORS
    try:
        engine = Engine.from_folder(args.model, EngineOptions(
            dtype=args.dtype, page_size=args.page_size, cache_tokens=tokens, max_requests=args.max_requests,
            max_step_tokens=tokens))           # a request may grow to the pool's size or the model's position limit
        replay(engine, sys.stdin, args.out, report)
    except USER_ERRORS as e:                       # what the input or the model folder can cause: one line, no trace
        sys.stderr.write(f"trace_run: error: {type(e).__name__}: {e}\n")
        return 1
    return 0
