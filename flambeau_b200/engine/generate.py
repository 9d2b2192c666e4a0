"""The Python entry point: token ids in, generated token ids out.

`generate()` is the call a user makes; `Generator` keeps an engine alive
between calls.  Option names follow the reference's command line where it has
them (crates/cli/src/main.rs:57-71 `infer`: --model, --prompt, --max-tokens,
--devices; :124-229 `serve`: --inflight-slots, --prefill-ubatch,
--prefill-chunk-tokens, --paged-kv, --ctx-cap) and its sampling fields
(crates/runtime/src/sampling.rs:39-50).
"""
from __future__ import annotations

import torch

from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .scheduler import Scheduler
from .step import Engine, EngineOptions


class EngineExecutor:
    """What the scheduler drives: the engine's step followed by the sampler."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.cache = engine.cache
        self.max_request_tokens = engine.max_seq_len       # the scheduler ends a request there with 'length'
        self.sampler = Sampler(engine.runtime.device, engine.options.max_requests)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def run(self, entries, sampled) -> list:
        handle = self.launch(entries, sampled)
        return self.collect(handle) if handle is not None else []

    def launch(self, entries, sampled, feed=None, pending: int = 0):
        """Queue a step and the sampling of its wanted rows without waiting for anything.  `feed`: the handle of
        the step before, whose sampled tokens (in the order of `entries`) are this step's token ids; `pending`:
        how many tokens of each sampled request the host has not seen yet (they count for the draw index)."""
        logits = self.engine.step(entries, token_feed=feed.tokens if feed is not None else None)
        self.h2d_bytes += self.engine.last_batch.h2d_bytes
        if not sampled:
            return None
        rows = [(r.params, r.generated, len(r.generated) + pending) for r in sampled]
        handle = self.sampler.launch(logits, rows)
        self.h2d_bytes += 8 * 4 * len(rows)
        self.d2h_bytes += 4 * len(rows)
        return handle

    def collect(self, handle) -> list:
        return self.sampler.collect(handle)

    def can_run_ahead(self, sampled) -> bool:
        """A step may be queued before the tokens of the step before it are known if sampling does not need them
        on the host (penalties count the generated tokens there)."""
        return all(not r.params.has_penalties for r in sampled)

    def finish(self, request_id) -> None:
        self.engine.finish(request_id)


class Generator:
    def __init__(self, engine: Engine, *, prefill_chunk_tokens: int = 2048, prefill_ubatch: int | None = None,
                 inflight_slots: int | None = None, run_ahead: bool = True):
        self.engine = engine
        self.run_ahead = run_ahead             # queue decode steps before the tokens of the step before are read
        self.executor = EngineExecutor(engine)
        self.prefill_chunk_tokens = prefill_chunk_tokens
        self.token_budget = min(prefill_ubatch or engine.options.max_step_tokens, engine.options.max_step_tokens)
        self.inflight_slots = min(inflight_slots or engine.options.max_requests, engine.options.max_requests)
        self.last_scheduler = None

    def generate(self, prompts, params=None) -> list:
        """prompts: list of token-id lists; params: one SamplingParams for all or one per prompt.
        Returns the generated token ids of each prompt, in order."""
        if params is None:
            params = SamplingParams()
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        if len(plist) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        sched = Scheduler(self.executor, token_budget=self.token_budget, prefill_chunk=self.prefill_chunk_tokens,
                          max_running=self.inflight_slots, run_ahead=self.run_ahead)
        reqs = [sched.add(i, p, sp) for i, (p, sp) in enumerate(zip(prompts, plist))]
        sched.run()
        self.engine.runtime.check_status("generate")
        self.last_scheduler = sched
        return [r.generated for r in reqs]


def generate(model, prompts, *, max_tokens: int = 64, temperature: float = 0.0, top_p=None, top_k=None, min_p=None,
             repetition_penalty: float = 1.0, presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
             logit_bias=None, seed: int = 0, stop_token_ids=(), dtype: str = "bfloat16", devices: str = "cuda:0",
             inflight_slots: int = 4, prefill_ubatch: int = 2048, prefill_chunk_tokens: int = 2048,
             paged_kv: int | None = None, ctx_cap: int | None = None, page_size: int = 16) -> list:
    """Generate `max_tokens` tokens for each prompt (lists of token ids).

    model: a folder with config.json and model.safetensors, or an Engine to reuse.
    temperature <= 0 is greedy.  Request i draws with seed `seed + i`.
    prefill_ubatch / prefill_chunk_tokens: the most rows of one step and the longest portion of a prompt in it.
    The reference's defaults are 512 for both, chosen for GPUs of 1 TB/s; here they are 2,048: on a B200 a step of
    2,048 rows runs the products at 1.2 to 1.4 PFLOP/s where one of 512 rows reaches 0.6 to 1.0, and takes about as
    long (27 ms for the 7B shape) as a 512-row step does there.
    paged_kv: number of cache pages (default: enough for `inflight_slots` requests of the longest prompt
    plus max_tokens); ctx_cap: the most tokens one request may hold, prompt and generated together: a request
    that reaches it ends there, one whose prompt is longer gets no tokens."""
    if max_tokens < 0:
        raise ValueError("max_tokens must not be negative")
    longest = max((len(p) for p in prompts), default=1) + max_tokens
    if ctx_cap:
        longest = min(longest, ctx_cap)
    per_request = -(-longest // page_size) * page_size
    if isinstance(model, Engine):
        engine = model
    else:
        if devices.startswith("cuda") is False:
            raise ValueError(f"devices = {devices!r}: this engine runs on one CUDA device, e.g. cuda:0")
        cache_tokens = paged_kv * page_size if paged_kv else inflight_slots * per_request
        engine = Engine.from_folder(model, EngineOptions(
            dtype=dtype, page_size=page_size, cache_tokens=cache_tokens, max_requests=inflight_slots,
            max_step_tokens=max(prefill_ubatch, inflight_slots), max_seq_len=longest, device=devices))
    gen = Generator(engine, prefill_chunk_tokens=prefill_chunk_tokens, prefill_ubatch=prefill_ubatch,
                    inflight_slots=inflight_slots)
    params = [SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                             repetition_penalty=repetition_penalty, presence_penalty=presence_penalty,
                             frequency_penalty=frequency_penalty, logit_bias=logit_bias, seed=seed + i,
                             max_tokens=max_tokens, stop_token_ids=stop_token_ids) for i in range(len(prompts))]
    return gen.generate(prompts, params)
