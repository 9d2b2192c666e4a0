"""The step function: a batch of (request, its next tokens) in, logits at the
wanted places out.

One step runs exactly the tokens it is given, as one batch, against the cache
that earlier steps left: portions of prompts of any length beside single
decoded tokens, in any mix.  The reference has three shapes of step (one
prompt portion, N decode tokens, or exactly one portion plus decode tokens;
crates/forward/src/runtime/mod.rs:188-258, ctx.rs:42-94); here a decoded token
is just a portion of length one and any number of portions may share a step.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from ..cache.manager import CacheManager
from ..kernels import library, ops
from .batch import BatchBuffers, BatchError, Entry, StepBatch
from .runtime import Runtime, Workspace


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"            # 'bfloat16' (serving kernels) or 'float32' (true 32-bit everywhere)
    page_size: int = 16                # tokens per cache page (crates/forward/src/core/scratch.rs:293)
    cache_tokens: int = 4096           # tokens the page pool of each group can hold
    max_requests: int = 8              # live requests (state slots, block-table rows)
    max_step_tokens: int = 2048        # rows of one step
    max_seq_len: Optional[int] = None  # longest request; default: the pool size or the model's position limit
    device: str = "cuda:0"
    cuda_graphs: bool = True           # replay steps of single decoded tokens from a captured CUDA graph


class StepContext:
    """What parts see during one step."""

    def __init__(self, engine, batch: StepBatch):
        self.engine = engine
        self.runtime = engine.runtime
        self.batch = batch
        self.n_tokens = batch.n_tokens
        self.ws = engine.runtime.ws
        self.shared: dict = {}              # per-step memo shared between layers (rotary tables, work lists)
        self.normed = self.delta = self.delta_slabs = None
        self.max_slabs = 1                  # how many split-K slabs a product may leave for the next kernel to add
        self.pending_slabs = 1
        self.stream_x = None                # the residual stream of the block that is running (set by the block)
        self.l2_hints = engine.l2_hints

    def open_stream(self, width: int):
        """Allocate what the blocks of a step share: the float32 residual stream (returned), the buffer for
        normalised rows (ctx.normed) and the float32 output of mixers and feed-forwards (ctx.delta).  A part's
        last product may leave its split-K shares in up to ctx.max_slabs slabs (ctx.delta_slabs, ctx.delta being
        the first), which the next norm adds: many for steps of few rows (decoding), where the split fills the
        GPU, a few for long portions, where it balances the last wave of a deep product."""
        n = self.n_tokens
        x = self.step_alloc((n, width), torch.float32)
        self.normed = self.step_alloc((n, width), self.runtime.dtype)
        self.max_slabs = 8 if n <= 64 else 4       # (16 for the fewest rows was measured: the kernels that add the
                                                   # shares take them four at a time, and a ninth costs a round trip)
        self.delta_slabs = self.step_alloc((self.max_slabs, n, width), torch.float32)
        self.delta = self.delta_slabs[0]
        self.pending_slabs = 1
        return x

    def to_stream(self, linear, a) -> None:
        """The last product of a mixer or a feed-forward, whose result belongs on the residual stream: added to
        the stream by the product's own epilogue where that is possible (ctx.pending_slabs = 0: nothing is left to
        add), else left in ctx.delta_slabs for the next norm to add (ctx.pending_slabs = how many slabs)."""
        if self.stream_x is not None and linear.add_into(self, a, self.stream_x):
            self.pending_slabs = 0
        else:
            self.pending_slabs = linear.slabs(self, a, self.delta_slabs)

    def step_alloc(self, shape, dtype):
        """Scratch that lives until the step ends (ctx.ws allocations end with their scope)."""
        return self.engine.step_ws.alloc(shape, dtype)

    def cache(self, call: int):
        return self.engine.cache.view(call, self.batch.tables, self.batch.table_bases)

    def logits(self, n_out: int, vocab: int):
        return self.engine.logits_buffer(n_out, vocab)


class Engine:
    """A model, its cache and the step function."""

    def __init__(self, model, options: EngineOptions):
        self.model = model
        self.options = options
        self.runtime: Runtime = model.runtime
        rt = self.runtime
        limit = options.max_seq_len or min(options.cache_tokens, model.spec.max_positions or options.cache_tokens)
        if model.spec.max_positions and limit > model.spec.max_positions:
            raise ValueError(f"max_seq_len = {limit} is more than the {model.spec.max_positions} positions the "
                             f"model's configuration allows")
        self.max_seq_len = int(limit)
        self.cache = CacheManager(model.cache_plans(), max_tokens=options.cache_tokens, page_size=rt.page_size,
                                  max_requests=options.max_requests, device=rt.device, dtype=rt.dtype,
                                  max_seq_len=self.max_seq_len, max_step_tokens=options.max_step_tokens)
        self.buffers = BatchBuffers(rt.device, options.max_step_tokens, options.max_requests, self.cache.n_groups,
                                    self.cache.table_pages)
        self.step_ws = Workspace(rt.device, 1 << 22)
        self._logits = None
        self._copied = torch.cuda.Event()
        self._copy_pending = False
        self.steps_run = 0
        self.last_batch: Optional[StepBatch] = None
        self._graphs: dict = {}            # step shape -> captured graph (or the count of eager runs so far)
        self.use_graphs = bool(options.cuda_graphs) and model.graph_safe()
        # the decode attention kernel fetches the start of the output projection's weights into L2 at its end
        self.l2_hints = options.dtype == "bfloat16" and os.environ.get("FLAMBEAU_L2_HINTS", "1") != "0"
        self.graph_replays = 0

    # ---- construction ----------------------------------------------------------
    @classmethod
    def from_folder(cls, folder, options: EngineOptions | None = None, **kw) -> "Engine":
        from .. import models  # noqa: F401  (registers the built-in architectures)
        from ..weights.loader import load_model
        options = options or EngineOptions(**kw)
        rt = Runtime(options.device, options.dtype, options.page_size)
        return cls(load_model(folder, rt), options)

    @classmethod
    def from_config(cls, config, seed: int = 0, options: EngineOptions | None = None, **kw) -> "Engine":
        """Random weights generated on the device (no model folder)."""
        from .. import models  # noqa: F401
        from ..config.registry import resolve
        from ..models.decoder import DecoderModel
        from ..weights.random_init import fill_random_on_device
        options = options or EngineOptions(**kw)
        rt = Runtime(options.device, options.dtype, options.page_size)
        model = DecoderModel(resolve(config.architecture).build_spec(config), rt)
        model.config = config
        fill_random_on_device(model, seed)
        return cls(model, options)

    # ---- buffers -----------------------------------------------------------------
    def logits_buffer(self, n_out: int, vocab: int) -> torch.Tensor:
        if self._logits is None or self._logits.shape[0] < n_out or self._logits.shape[1] != vocab:
            rows = max(n_out, self.options.max_requests)
            self._logits = torch.empty((rows, vocab), dtype=torch.float32, device=self.runtime.device)
        return self._logits[:n_out]

    # ---- running a packed batch: eagerly, or by replaying a captured graph -----------------------------
    def _forward(self, batch: StepBatch):
        self.runtime.ws.reset()
        self.step_ws.reset()
        return self.model.forward(StepContext(self, batch))

    def _graph_key(self, batch: StepBatch):
        """Steps of single decoded tokens repeat with the same shape; everything that differs between them
        (tokens, positions, block tables, wanted rows) lives in the descriptor buffers, whose addresses are
        fixed.  The key holds what is baked into kernel arguments: the number of sequences and wanted rows.
        Context lengths are not in it: the attention kernel splits the key range on the device, from the
        descriptor, with a grid that does not depend on them."""
        if not self.use_graphs or batch.max_q_len != 1:
            return None
        if batch.n_out not in (0, batch.n_seqs):
            return None
        return (batch.n_seqs, batch.n_out)

    def _run(self, batch: StepBatch):
        key = self._graph_key(batch)
        if key is None:
            return self._forward(batch)
        entry = self._graphs.get(key, 0)
        if isinstance(entry, int):
            if entry < 1:                               # first time: run eagerly (lazy allocations, attributes)
                self._graphs[key] = entry + 1
                return self._forward(batch)
            try:
                entry = self._capture(batch, key)
            except Exception as exc:                    # a part that cannot be captured after all: run eagerly
                import warnings
                warnings.warn(f"CUDA graph capture failed ({exc}); steps run eagerly from now on")
                self.use_graphs = False
                torch.cuda.synchronize()
                return self._forward(batch)
        graph, logits, _keep, n_kernels = entry
        graph.replay()
        library.LAUNCHES[0] += n_kernels                # the launches the graph replays
        self.graph_replays += 1
        return logits

    def _capture(self, batch: StepBatch, key):
        rt = self.runtime
        # a replay serves any context length: a part that sizes something by the longest context sees the limit
        real = batch.max_kv_len
        batch.max_kv_len = self.max_seq_len
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        launches_before = library.LAUNCHES[0]
        rt.ws.frozen = self.step_ws.frozen = True
        try:
            with torch.cuda.graph(graph):
                logits = self._forward(batch)
        finally:
            rt.ws.frozen = self.step_ws.frozen = False
            batch.max_kv_len = real
        # the graph holds raw addresses: keep the buffers it wrote into and read from alive with it
        keep = (rt.ws.buffer, self.step_ws.buffer, self._logits)
        n_kernels = library.LAUNCHES[0] - launches_before
        library.LAUNCHES[0] = launches_before           # capturing launched nothing
        entry = (graph, logits, keep, n_kernels)
        self._graphs[key] = entry
        return entry

    # ---- requests ----------------------------------------------------------------
    def admit(self, request_id):
        return self.cache.admit(request_id)

    def finish(self, request_id) -> None:
        self.cache.release(request_id)

    def is_live(self, request_id) -> bool:
        return request_id in self.cache.requests

    def snapshot(self, request_id):
        """What the request holds in the cache (keys, values, fixed-size state, length) as host tensors."""
        return self.cache.snapshot(request_id)

    def restore(self, request_id, snapshot) -> None:
        """Make `request_id` live again from a snapshot; its next step continues at the snapshot's length."""
        self.cache.restore(request_id, snapshot)

    # ---- the step ------------------------------------------------------------------
    def step(self, entries: list, end=(), token_feed: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run `entries` (Entry or (request_id, tokens, want) tuples) as one batch.

        `token_feed` (device int32, one id per entry, every entry a single token): the token ids are taken from
        it on the device, in stream order, instead of from the entries; this is how a decode step is queued
        before the host has seen the tokens the step before it sampled.

        Unknown request ids are admitted.  Returns float32 logits [wanted, vocab] on the device, in the
        order of the entries and of each entry's `want` (None if nothing is wanted); the tensor is
        overwritten by the next step.  Requests in `end` give back what they hold after the step.
        Raises cache.pages.OutOfPages before anything runs if the pages do not suffice."""
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        cache = self.cache
        logits = None
        if entries:
            if token_feed is not None and (any(len(e.tokens) != 1 for e in entries)
                                           or token_feed.numel() < len(entries)):
                raise BatchError("a token feed needs single-token entries and one id per entry")
            admitted = []
            try:
                for e in entries:
                    if e.request_id not in cache.requests:
                        cache.admit(e.request_id)
                        admitted.append(e.request_id)
                needs = [(e.request_id, len(e.tokens)) for e in entries]
                for rid, k in needs:
                    if cache.length(rid) + k > self.max_seq_len:
                        raise BatchError(f"request {rid!r} would reach {cache.length(rid) + k} tokens; "
                                         f"the engine was built for {self.max_seq_len} per request")
                cache.reserve_all(needs)
                if self._copy_pending:
                    self._copied.synchronize()      # the staging buffers are free to be rewritten
                batch = self.buffers.build(entries, cache, self.model.vocab_size)
                if token_feed is not None:
                    self.buffers.d_rows[0, :batch.n_seqs].copy_(token_feed[:batch.n_seqs])
                self._copied.record()
                self._copy_pending = True
                logits = self._run(batch)
            except Exception:
                # The step did not run to its end on the host (a bad entry, no pages, a launch that was refused):
                # requests that this step brought in leave again, with what was reserved for them; lengths have
                # not advanced, and pages reserved beyond a live request's length are taken by its next step.
                for rid in admitted:
                    if rid in cache.requests:
                        cache.release(rid)
                raise
            cache.commit_all(needs)
            self.last_batch = batch
            self.steps_run += 1
        for rid in end:
            if rid in cache.requests:
                cache.release(rid)
        return logits
