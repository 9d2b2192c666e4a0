#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200: ONE JSON line on standard output.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 7b|nemo12b|small24b] [--only headline|mixed|shapes] [--batch B] [--context C] [--layers L]

The same program as `flambeau bench`; what it measures, how, and the keys of the line are described in
flambeau_b200/measure/bench.py.  Default run: the Mistral-7B-v0.1 shape with random bfloat16 weights, decode at
batch 8 with 8,192 tokens of context a sequence (`value`, and `e2e` through the scheduler's loop with host token
ids in and out), batch 1 and 64, a 2,048-token prefill, rooflines against MEASURED_PEAKS.json, per-kernel times,
a correctness check of the benchmarked attention geometry, the Mistral-Nemo-12B mixed workload through the
scheduler and the Mistral-Small-24B shape; about 20 s.  For more than one GPU it prints one line saying that
the engine runs on one GPU and exits with 2.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from flambeau_b200.measure.bench import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
