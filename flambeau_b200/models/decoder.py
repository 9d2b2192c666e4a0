"""A decoder-only model as data plus parts: embedding, a list of blocks, the
order in which they run, a final norm and an output head.

Nothing here is specific to an architecture; an architecture only supplies the
ModelSpec.  The part order of one step is the reference's
(crates/forward/README.md:18-39): embed, the layer calls, then final norm and
head on the wanted rows only (crates/forward/src/core/composites/output_head.rs:32-57).
"""
from __future__ import annotations

import torch

from ..cache.manager import CallPlan
from ..parts.block import ResidualStream
from ..parts.spec import ModelSpec, build_part


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self.embedding = build_part(spec.embedding, runtime)
        self.layers = [build_part(s, runtime) for s in spec.layers]
        self.order = list(spec.order)
        self.final_norm = build_part(spec.final_norm, runtime)
        self.head = build_part(spec.head, runtime)

    # ---- weights -----------------------------------------------------------
    def parts(self):
        return [self.embedding, *self.layers, self.final_norm, self.head]

    def tensor_specs(self) -> dict:
        specs = {}
        for p in self.parts():
            for name, ts in p.tensor_specs().items():
                if name in specs and specs[name].shape != ts.shape:
                    raise ValueError(f"two parts want tensor '{name}' with different shapes")
                specs[name] = ts
        return specs

    def bind(self, tensors: dict) -> None:
        for p in self.parts():
            p.bind(tensors)

    def graph_safe(self) -> bool:
        return all(p.all_graph_safe() for p in self.parts())

    def step_weight_bytes(self) -> int:
        """Bytes of weights one step reads: every layer call's weights once, the final norm and the head."""
        total = self.final_norm.weight_bytes() + self.head.weight_bytes()
        for call in self.order:
            total += self.layers[call.layer].weight_bytes()
        return total

    # ---- what the cache manager must provide ---------------------------------
    def cache_plans(self) -> list:
        plans = []
        for call in self.order:
            mixer = self.layers[call.layer].mixer
            plans.append(CallPlan(kv=mixer.cache_requirement(), state=mixer.state_requirement(),
                                  cache_from=call.cache_from))
        return plans

    # ---- one step -------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor | None:
        """Runs the rows of ctx.batch; returns float32 logits [n_out, vocab] (None when nothing is wanted)."""
        rt, b = self.runtime, ctx.batch
        n = b.n_tokens
        x = ctx.open_stream(self.hidden_size)
        self.embedding.forward(ctx, b.token_ids[:n], x)
        stream = ResidualStream(x)
        for ci, call in enumerate(self.order):
            self.layers[call.layer].forward(ctx, stream, ci)
        if b.n_out == 0:
            return None
        h = ctx.step_alloc((b.n_out, self.hidden_size), rt.dtype)
        self.final_norm.add_norm(ctx, stream.x, stream.pending, h, rows=b.out_rows[:b.n_out],
                                 n_partials=stream.pending_slabs)
        logits = ctx.logits(b.n_out, self.vocab_size)
        self.head.forward(ctx, h, logits)
        return logits
