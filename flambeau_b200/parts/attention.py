"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import KVRequirement, Mixer, TensorSpec
from .linear import Linear, concat_rows
from .spec import PartSpec, build_part, register_part


class PagedAttention(Mixer):
    """q, k, v = h Wq^T, h Wk^T, h Wv^T (no bias); position encoding on q and k
    after the projection and before the cache write; every query at position p
    attends to the cached keys [max(0, p-W+1), p] of its request (all of [0, p]
    when window == 0) with scores scale * q.k; o = a Wo^T.
    crates/forward/src/core/composites/standard_attn.rs:197-286 (projections),
    :355-399 (rotary), :418-420 (scale), :1261-1302 (output projection).

    Sizes are parameters: `num_heads * head_dim` need not equal `width`.
    `qk_norm` (optional, a norm PartSpec of width head_dim): a norm over every
    head of q and of k between the projection and the rotation, with weights
    `<prefix>q_norm.weight` and `<prefix>k_norm.weight` (the optional
    attn_q_norm / attn_k_norm of crates/forward/src/ctx.rs:368-369; the
    architecture built here has none).
    `distance_slopes` (optional, one number per query head): slope * (key
    position - query position) is added to every scaled score, a linear
    penalty on distance that a position scheme without rotation can be built
    from (the architecture built here has none; portions of prompts then run
    on the mma.sync kernel, which has the hook)."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 window: int = 0, position: PartSpec | None = None, scale: float | None = None,
                 init_std: float = 0.02, qk_norm: PartSpec | None = None, distance_slopes=None):
        super().__init__(runtime, prefix)
        self.width, self.nh, self.nkv, self.hd = int(width), int(num_heads), int(num_kv_heads), int(head_dim)
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} query heads are not a multiple of {self.nkv} key/value heads")
        self.window = int(window or 0)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        self.position = build_part(position, runtime) if position is not None else None
        self.q_norm = self.k_norm = None
        if qk_norm is not None:
            self.q_norm = build_part(PartSpec(qk_norm.category, qk_norm.kind, qk_norm.params, prefix + "q_norm."), runtime)
            self.k_norm = build_part(PartSpec(qk_norm.category, qk_norm.kind, qk_norm.params, prefix + "k_norm."), runtime)
        self.init_std = init_std
        self.distance_slopes = None
        if distance_slopes is not None:
            slopes = [float(x) for x in distance_slopes]
            if len(slopes) != self.nh:
                raise ValueError(f"{len(slopes)} distance slopes for {self.nh} query heads")
            self.distance_slopes = torch.tensor(slopes, dtype=torch.float32,
                                                device=runtime.device if runtime is not None else "cpu")
        self.qw, self.kvw = self.nh * self.hd, self.nkv * self.hd
        self.qkv = self.o = None

    def children(self):
        return [p for p in (self.position, self.q_norm, self.k_norm) if p is not None]

    def cache_requirement(self):
        return KVRequirement(self.nkv, self.hd, self.window)

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        return {
            p + "q_proj.weight": TensorSpec((self.qw, self.width), init=init),
            p + "k_proj.weight": TensorSpec((self.kvw, self.width), init=init),
            p + "v_proj.weight": TensorSpec((self.kvw, self.width), init=init),
            p + "o_proj.weight": TensorSpec((self.width, self.qw), init=init),
        }

    def own_bind(self, tensors):
        p = self.prefix
        self.qkv = Linear(concat_rows([tensors[p + "q_proj.weight"], tensors[p + "k_proj.weight"],
                                       tensors[p + "v_proj.weight"]]))
        self.o = Linear(tensors[p + "o_proj.weight"])

    def own_weights(self):
        return [self.qkv.weight, self.o.weight]

    def forward(self, ctx, h, out, call):
        n = ctx.n_tokens
        rt = self.runtime
        cache = ctx.cache(call)
        with ctx.ws.scope():
            # the projection stays float32 until after the rotation, so q and k are rounded once
            pos = self.position
            fused = pos is None or getattr(pos, "fused_with_cache_write", False)
            # the fused rotary kernel adds split-K shares of the projection itself; a position encoding with a
            # rotate() of its own gets whole rows
            if self.q_norm is None:
                qkv_slabs = ctx.ws.alloc((ctx.max_slabs if fused else 1, n, self.qw + 2 * self.kvw), torch.float32)
                parts = self.qkv.slabs(ctx, h, qkv_slabs)
                stride = qkv_slabs.stride(0)
                qkv = qkv_slabs[0]
                q_in = qkv[:, :self.qw]
                k = qkv[:, self.qw:self.qw + self.kvw]
                v = qkv[:, self.qw + self.kvw:]
            else:
                # un-fused: three products from row slices of the stacked weight, so that the heads of q and of k
                # lie as rows of their own; each head is normalised, then everything goes on as before
                parts, stride = 1, 0
                w = self.qkv.weight
                qn, kn = ctx.ws.alloc((n, self.qw), torch.float32), ctx.ws.alloc((n, self.kvw), torch.float32)
                q_in, k = ctx.ws.alloc((n, self.qw), torch.float32), ctx.ws.alloc((n, self.kvw), torch.float32)
                v = ctx.ws.alloc((n, self.kvw), torch.float32)
                ops.linear(h, w[:self.qw], qn, ctx)
                ops.linear(h, w[self.qw:self.qw + self.kvw], kn, ctx)
                ops.linear(h, w[self.qw + self.kvw:], v, ctx)
                self.q_norm.normalize(ctx, qn.view(n * self.nh, self.hd), q_in.view(n * self.nh, self.hd))
                self.k_norm.normalize(ctx, kn.view(n * self.nkv, self.hd), k.view(n * self.nkv, self.hd))
            q = ctx.ws.alloc((n, self.qw), rt.dtype)
            b = ctx.batch
            if fused:
                cos, sin = pos.prepare(ctx) if pos is not None else (None, None)
                half = pos.half if pos is not None else 0
                ops.rope_kv_write(q_in, q, k, v, cos, sin, half, b.positions, b.row_seq, cache.block_table,
                                  cache.k_pool, cache.v_pool, cache.page_size, self.nh, self.nkv, self.hd,
                                  cache.writable, rt.status, n_partials=parts, partial_stride=stride,
                                  table_base=cache.table_base)
            else:
                pos.rotate(ctx, q_in, k if cache.writable else None)
                ops.rope_kv_write(q_in, q, k, v, None, None, 0, b.positions, b.row_seq, cache.block_table,
                                  cache.k_pool, cache.v_pool, cache.page_size, self.nh, self.nkv, self.hd,
                                  cache.writable, rt.status, table_base=cache.table_base)
            a = ctx.ws.alloc((n, self.qw), rt.dtype)
            # few rows: the attention kernel fetches the start of the output projection's weights into L2 at its end
            hint = self.o.weight if ctx.l2_hints and n <= 64 else None
            ops.paged_attention(ctx, q, a, cache, self.nh, self.nkv, self.hd, self.window, self.scale,
                                next_weight=hint, score_slopes=self.distance_slopes)
            ctx.to_stream(self.o, a)


register_part("mixer", "attention", PagedAttention)
