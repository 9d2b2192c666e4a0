"""Interfaces of the parts a layer is put together from.

A part knows its own sizes and constants (they are constructor arguments) and
never which model it sits in.  Every part

  * lists the tensors it wants from the weight file (`tensor_specs`),
  * receives them, already on the device, in `bind`,
  * and does its work in a method that takes the step context first.

Categories and the method each must have:

  norm           add_norm(ctx, x, delta, out, rows=None, n_partials=1)
                 x: float32 stream [n, width], updated in place with delta when
                 rows is None; out: normalised rows in the engine dtype.
                 normalize(ctx, x, out): the norm of every row of x alone.
  position       prepare(ctx) -> per-step tables (memoised in ctx.shared);
                 rotate(ctx, q, k) in place on [n, heads*head_dim] views.
  mixer          forward(ctx, h, out, call); cache_requirement() -> KVRequirement | None;
                 state_requirement() -> StateRequirement | None.
  feed_forward   forward(ctx, h, out).
  block          forward(ctx, stream, call); mixer and feed_forward attributes.
  embedding      forward(ctx, token_ids, x).
  head           forward(ctx, h_rows, logits).

`ctx` is an engine.step.StepContext: the batch descriptor on the device, the
cache views of the running layer call, the scratch arena and a per-step memo.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .spec import TensorSpec


@dataclass(frozen=True)
class KVRequirement:
    """A mixer that keeps keys and values: layers with equal requirements share
    a cache group (one page-id space, one block table per request)."""
    kv_heads: int
    head_dim: int
    window: int = 0          # 0 = all earlier keys stay live; W > 0 = only the last W


@dataclass(frozen=True)
class StateRequirement:
    """A mixer that keeps a fixed-size state per request: `shape` elements of
    `dtype` ('float32' or 'engine') in the request's slot, zeroed on admission."""
    shape: tuple
    dtype: str = "float32"


class Part:
    category = "part"
    # A part whose work in a step is kernels on the current stream with arguments that depend only on the step's
    # shape may be captured in a CUDA graph and replayed.  A part that reads the batch on the host, copies from
    # host memory or allocates must leave this False; the engine then runs steps with it eagerly.
    graph_safe = False

    def __init__(self, runtime=None, prefix: str = ""):
        self.runtime = runtime
        self.prefix = prefix

    # -- weights ------------------------------------------------------------
    def tensor_specs(self) -> dict:
        """full tensor name -> TensorSpec, children included."""
        specs = dict(self.own_tensor_specs())
        for child in self.children():
            specs.update(child.tensor_specs())
        return specs

    def own_tensor_specs(self) -> dict:
        return {}

    def children(self) -> list:
        return []

    def bind(self, tensors: dict) -> None:
        """Take the device tensors this part declared (by full name)."""
        self.own_bind(tensors)
        for child in self.children():
            child.bind(tensors)

    def own_bind(self, tensors: dict) -> None:
        pass

    def weight_bytes(self) -> int:
        """Bytes of weights this part reads in one step (children included)."""
        return sum(t.numel() * t.element_size() for t in self.own_weights()) + \
            sum(c.weight_bytes() for c in self.children())

    def own_weights(self) -> list:
        return []

    def all_graph_safe(self) -> bool:
        return bool(self.graph_safe) and all(c.all_graph_safe() for c in self.children())


class Mixer(Part):
    category = "mixer"

    def cache_requirement(self) -> Optional[KVRequirement]:
        return None

    def state_requirement(self) -> Optional[StateRequirement]:
        return None

    def forward(self, ctx, h, out, call) -> None:
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, ctx, h, out) -> None:
        raise NotImplementedError


class Norm(Part):
    category = "norm"

    def add_norm(self, ctx, x, delta, out, rows=None, n_partials: int = 1) -> None:
        raise NotImplementedError

    def normalize(self, ctx, x, out) -> None:
        """out = the norm of every row of x (float32 [rows, width], contiguous), nothing added, x unchanged:
        what a mixer's query/key norm calls with rows = tokens x heads and width = the head size."""
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"

    def prepare(self, ctx):
        return None

    def rotate(self, ctx, q, k) -> None:
        raise NotImplementedError


__all__ = ["KVRequirement", "StateRequirement", "Part", "Mixer", "FeedForward", "Norm", "PositionEncoding",
           "TensorSpec"]
