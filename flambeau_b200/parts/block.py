"""How a layer arranges its norms, mixer and feed-forward around the stream."""
from __future__ import annotations

from .base import Part
from .spec import PartSpec, build_part, register_part


class ResidualStream:
    """The float32 stream x [n, width] plus the last part's output that has
    not been added yet (`pending`): the next norm adds it while it normalises,
    so the add costs no pass of its own.  `pending_slabs` > 1 says that the
    output is a sum of that many float32 slabs (split-K shares of the part's last
    product, ctx.delta_slabs[0..k)), which the norm adds as well; 0 says that the
    part's last product has added its result to x itself (ctx.to_stream), so the
    norm has nothing to add."""

    def __init__(self, x, pending=None, pending_slabs: int = 1):
        self.x, self.pending, self.pending_slabs = x, pending, pending_slabs


class PreNormBlock(Part):
    """x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x))
    (crates/models/qwen35-v2/src/model.rs:25-42)."""
    graph_safe = True
    category = "block"

    def __init__(self, runtime=None, prefix="", *, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec):
        super().__init__(runtime, prefix)
        self.mixer = build_part(mixer, runtime)
        self.feed_forward = build_part(feed_forward, runtime)
        self.mixer_norm = build_part(mixer_norm, runtime)
        self.feed_forward_norm = build_part(feed_forward_norm, runtime)

    def children(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, ctx, stream: ResidualStream, call) -> None:
        h, delta = ctx.normed, ctx.delta
        ctx.stream_x = stream.x
        self.mixer_norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs)
        ctx.pending_slabs = 1                 # a part that leaves split-K shares in ctx.delta_slabs says how many
        self.mixer.forward(ctx, h, delta, call)
        stream.pending, stream.pending_slabs = delta, ctx.pending_slabs
        self.feed_forward_norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs)
        ctx.pending_slabs = 1
        self.feed_forward.forward(ctx, h, delta)
        stream.pending, stream.pending_slabs = delta, ctx.pending_slabs
        ctx.stream_x = None                   # another kind of block decides for itself whether parts may add to its stream


register_part("block", "pre_norm", PreNormBlock)
