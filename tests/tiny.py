"""Tiny configurations, model folders and replay schedules shared by the tests.

Two configurations that differ in every size and option:
  A: 2 layers, width 64, 4 heads / 2 kv heads, head 16, inner 128, vocab 256, theta 1e4, window 16, eps 1e-5, untied
  B: 3 layers, width 96, 8 heads / 1 kv head, head 24 (heads*head != width), inner 160, vocab 320, theta 1e6,
     no window, eps 1e-6, tied
"""
from __future__ import annotations

import json
import random
from pathlib import Path

import numpy as np
import torch

CONFIG_A = dict(architectures=["MistralForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
                sliding_window=16, rms_norm_eps=1e-5, tie_word_embeddings=False, hidden_act="silu")
CONFIG_B = dict(architectures=["MistralForCausalLM"], hidden_size=96, num_hidden_layers=3, num_attention_heads=8,
                num_key_value_heads=1, head_dim=24, intermediate_size=160, vocab_size=320, rope_theta=1000000.0,
                sliding_window=None, rms_norm_eps=1e-6, tie_word_embeddings=True, hidden_act="silu")
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B}

# tolerances, fixed up front: error relative to the largest |logit| of the plain implementation
TOL = {"float32": 1e-4, "bfloat16": 2e-2}


def tol_at_depth(dtype: str, layers: int) -> float:
    """The bound for a model of `layers` layers.  float32: the same 1e-4 at any depth.  bfloat16: the bound above
    is set for the tiny models (two and three layers); every layer rounds its normalised input, its queries, keys,
    values, attention output and feed-forward activation to 8 bits of mantissa, independent roundings whose effect
    on the logits adds in quadrature, so the bound grows with the square root of the depth beyond three layers."""
    if dtype == "float32":
        return TOL["float32"]
    return TOL["bfloat16"] * max(1.0, layers / 3.0) ** 0.5


def make_folder(folder, cfg: dict, seed: int, dtype: str, sharp: float | None = 0.2) -> Path:
    """A model folder with seeded random weights.  `sharp` redraws the query and key projections with that
    standard deviation, so that attention scores spread over several units and a wrong, missing or extra key
    changes the logits visibly (with N(0, 0.02) everywhere attention is almost uniform)."""
    from flambeau_b200.config.mistral import MistralConfig
    from flambeau_b200.weights.random_init import write_random_model
    from flambeau_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    folder = Path(folder)
    write_random_model(folder, MistralConfig.from_dict(cfg), seed=seed, dtype=dtype)
    if sharp:
        f = SafetensorsFile(folder / "model.safetensors")
        tensors = {n: f.tensor(n).clone() for n in f.names()}
        f.close()
        g = torch.Generator().manual_seed(seed * 7919 + 13)
        for n in sorted(tensors):
            if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
                t = tensors[n]
                tensors[n] = (torch.randn(t.shape, generator=g) * sharp).to(t.dtype)
        write_safetensors(folder / "model.safetensors", tensors)
    return folder


def random_requests(cfg: dict, lengths, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    return {f"r{i}": [int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)] for i, n in enumerate(lengths)}


# --------------------------------------------------------------------------
# schedules: lists of step records plus, per step, which (request, position) each written row is
# --------------------------------------------------------------------------

class Schedule:
    def __init__(self):
        self.steps: list = []
        self.rows: dict = {}            # step -> [(request id, position), ...] in file order

    def add(self, entries, end=()):
        step = len(self.steps)
        self.steps.append({"step": step, "entries": [
            {"id": rid, "tokens": toks, "want": want} for rid, toks, want, _ in entries], "end": list(end)})
        rows = []
        for rid, toks, want, pos0 in entries:
            rows += [(rid, pos0 + w) for w in want]
        if rows:
            self.rows[step] = rows
        return step

    def lines(self):
        return [json.dumps(s) for s in self.steps]

    def max_live_tokens(self, requests) -> int:
        """Most tokens held by live requests at any time, each rounded up to a multiple of 64."""
        live, held, best = {}, 0, 0
        for s in self.steps:
            for e in s["entries"]:
                live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
            best = max(best, sum(-(-v // 64) * 64 for v in live.values()))
            for rid in s["end"]:
                live.pop(rid, None)
        return best


def schedule_whole(requests) -> Schedule:
    s = Schedule()
    for rid, toks in requests.items():
        s.add([(rid, toks, list(range(len(toks))), 0)], end=[rid])
    return s


def schedule_tail(requests, tail: int = 32) -> Schedule:
    """Most of each request in one step, the last `tail` tokens one by one."""
    s = Schedule()
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        s.add([(rid, toks[:head], list(range(head)), 0)])
        for p in range(head, len(toks)):
            s.add([(rid, [toks[p]], [0], p)], end=[rid] if p == len(toks) - 1 else [])
        if head == len(toks):
            s.steps[-1]["end"] = [rid]
    return s


def schedule_portions(requests, sizes=(7, 2, 13, 3, 5, 2, 9, 4)) -> Schedule:
    """Portions of changing size, down to two tokens."""
    s = Schedule()
    for rid, toks in requests.items():
        p, i = 0, 0
        while p < len(toks):
            k = min(sizes[i % len(sizes)], len(toks) - p)
            last = p + k == len(toks)
            s.add([(rid, toks[p:p + k], list(range(k)), p)], end=[rid] if last else [])
            p, i = p + k, i + 1
    return s


def schedule_mixed(requests, seed: int, max_live: int = 4, prompt_fraction: float = 0.7) -> Schedule:
    """Up to `max_live` requests at a time: the first `prompt_fraction` of each request arrives in portions of
    random size (2..9), the rest one token a step, portions of some beside single tokens of others; a request
    may sit a step out.  New requests start as others end, so pages are used again."""
    rng = random.Random(seed)
    s = Schedule()
    waiting = list(requests.items())
    live = {}                                   # rid -> [tokens, next position, prompt length]
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, int(len(toks) * prompt_fraction))]
        entries, end = [], []
        for rid in list(live):
            toks, p, plen = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                        # left out of this step
            if p < plen:
                k = min(rng.randint(2, 9), plen - p)
                if plen - p - k == 1:
                    k += 1                      # never leave a one-token portion of the prompt
            else:
                k = 1
            entries.append((rid, toks[p:p + k], list(range(k)), p))
            live[rid][1] = p + k
            if p + k == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            s.add(entries, end=end)
    return s


def schedule_wild(cfg: dict, seed: int, max_live: int = 4):
    """A trace as a careless client writes it: ids that are used again for new requests after their `end`,
    requests ended before their last token, steps that want nothing or a few scattered places, portions of one
    token in mid-prompt, requests that sit steps out.  Returns (requests, schedule): the requests are keyed by a
    serial number, not by the reused id, and so are the schedule's rows."""
    rng = random.Random(seed)
    names = ["x", "y", "z", "w", "v"]
    s = Schedule()
    requests, live, serial = {}, {}, 0          # live: id -> [serial, tokens, next position, stop position]
    for _ in range(rng.randint(20, 70)):
        while len(live) < max_live and rng.random() < 0.5:
            name = rng.choice([n for n in names if n not in live])
            n_tok = rng.randint(1, 100)
            toks = [rng.randrange(cfg["vocab_size"]) for _ in range(n_tok)]
            stop = n_tok if rng.random() < 0.6 else rng.randint(1, n_tok)
            live[name] = [serial, toks, 0, stop]
            requests[serial] = toks
            serial += 1
        entries, rows = [], []
        for name in list(live):
            u, toks, p, stop = live[name]
            if p >= stop or (len(live) > 1 and rng.random() < 0.25):
                continue
            k = min(rng.choice([1, 1, 2, 3, 7, 20, 64]), stop - p)
            want = sorted(rng.sample(range(k), rng.randint(0, min(k, 4)))) if rng.random() < 0.8 else []
            entries.append({"id": name, "tokens": toks[p:p + k], "want": want})
            rows += [(u, p + w) for w in want]
            live[name][2] = p + k
        end = [name for name in list(live) if live[name][2] >= live[name][3] and rng.random() < 0.8]
        for name in end:
            del live[name]
        step = len(s.steps)
        s.steps.append({"step": step, "entries": entries, "end": end})
        if rows:
            s.rows[step] = rows
    return requests, s


def read_rows(out_dir, schedule: Schedule, vocab: int) -> dict:
    """(request id, position) -> float32 logits row, from the files a replay wrote."""
    got = {}
    for step, rows in schedule.rows.items():
        data = np.fromfile(Path(out_dir) / f"{step}.f32", dtype="<f4")
        assert data.size == len(rows) * vocab, f"step {step}: {data.size} floats for {len(rows)} rows"
        data = data.reshape(len(rows), vocab)
        for i, key in enumerate(rows):
            assert key not in got, f"row {key} written twice"
            got[key] = data[i]
    return got


def compare_rows(got: dict, want: dict, tol: float, what: str) -> float:
    """Every (request, position) of `want` (request -> [T, V] tensor) must be in `got` within tol * scale."""
    worst, worst_at = 0.0, None
    for rid, ref in want.items():
        ref = ref.numpy() if hasattr(ref, "numpy") else ref
        scale = float(np.abs(ref).max())
        for p in range(ref.shape[0]):
            assert (rid, p) in got, f"{what}: no logits for request {rid} position {p}"
            err = float(np.abs(got[(rid, p)].astype(np.float64) - ref[p]).max()) / scale
            assert np.isfinite(err), f"{what}: non-finite logits for request {rid} position {p}"
            if err > worst:
                worst, worst_at = err, (rid, p)
    print(f"[compare] {what}: worst error {worst:.3e} of the logit scale at {worst_at} (tolerance {tol:.0e})")
    assert worst <= tol, f"{what}: error {worst:.3e} of the logit scale at {worst_at} exceeds {tol:.0e}"
    return worst
