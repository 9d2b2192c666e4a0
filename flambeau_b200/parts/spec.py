"""Data that describes a model: which parts, with which sizes, in which order.

An architecture turns its typed configuration into a `ModelSpec`.  Nothing in
a spec is code: parts are named by (category, kind) and looked up in the part
registry when the model is built, so a model may use a different mixer or
feed-forward in every layer, run a layer twice, or let a layer read another
layer's cache, by changing data only.

The reference expresses the same thing with per-layer weight structs and a
layer-kind tag (crates/forward/src/ctx.rs:351-411, 530-533) and per-layer
cache geometry lists (crates/forward/src/core/scratch.rs:137-165).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part wants from the weight file.

    kind: 'float' tensors follow the engine's dtype rule (bfloat16 when
    serving unless stored in 32-bit; float32 in the 32-bit mode); 'int'
    tensors are kept as int32.
    init: how the random-weights mode fills it: ('normal', std),
    ('one_plus_normal', std) or ('ones',).
    alias_of: full name of another tensor that stands for this one when the
    file does not have it (tied embeddings).
    """
    shape: tuple
    kind: str = "float"
    init: tuple = ("normal", 0.02)
    alias_of: Optional[str] = None


@dataclass(frozen=True)
class PartSpec:
    """A part by category and kind, its parameters, and the prefix of its
    tensor names in the weight file."""
    category: str            # 'mixer' | 'feed_forward' | 'norm' | 'position' | 'block' | 'embedding' | 'head'
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run `layer`; if `cache_from` is given, the
    mixer writes nothing and reads the cache that the earlier call with that
    index in the order list owns."""
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: list            # list[PartSpec] of category 'block'
    order: list             # list[LayerCall]
    final_norm: PartSpec
    head: PartSpec
    max_positions: Optional[int] = None

    def validate(self) -> None:
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {call.layer}, the model has {len(self.layers)}")
            if call.cache_from is not None:
                if not 0 <= call.cache_from < i:
                    raise ValueError(f"order[{i}].cache_from = {call.cache_from} must name an earlier call")
                if self.order[call.cache_from].cache_from is not None:
                    raise ValueError(f"order[{i}].cache_from names a call that owns no cache")


# --------------------------------------------------------------------------
# part registry
# --------------------------------------------------------------------------

_PARTS: dict[tuple, Any] = {}


def register_part(category: str, kind: str, cls, *, replace: bool = False) -> None:
    key = (category, kind)
    if key in _PARTS and not replace:
        raise ValueError(f"part {category}/{kind} is already registered")
    _PARTS[key] = cls


def unregister_part(category: str, kind: str) -> None:
    _PARTS.pop((category, kind), None)


def part_class(category: str, kind: str):
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise ValueError(f"no {category} part of kind '{kind}'; known: {', '.join(known) or '(none)'}") from None


def build_part(spec: PartSpec, runtime):
    """Instantiate the registered class for `spec` with the spec's parameters."""
    cls = part_class(spec.category, spec.kind)
    return cls(runtime=runtime, prefix=spec.prefix, **spec.params)
