"""Rotary position encoding with split-half pairs."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import PositionEncoding
from .spec import register_part


class RotaryHalf(PositionEncoding):
    """Pair i in [0, rot/2) of a head is (x[i], x[i + rot/2]); its angle is
    pos * theta^(-2i/rot) (crates/kernels-hip/src/kernels/
    rope_neox_partial_f16.cu:39-52).  `rotary_dim` < head_dim leaves the tail
    of the head untouched.  The cos/sin tables of a step are computed once and
    shared by every layer that uses equal parameters."""
    graph_safe = True

    fused_with_cache_write = True      # the attention mixer may hand the tables to its fused kernel

    def __init__(self, runtime=None, prefix="", *, head_dim: int, theta: float, rotary_dim: int | None = None):
        super().__init__(runtime, prefix)
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.half = self.rotary_dim // 2
        self._inv_freq = None

    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            i = torch.arange(self.half, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rotary_dim)
            self._inv_freq = inv.to(self.runtime.device)
        return self._inv_freq

    def prepare(self, ctx):
        """(cos, sin), float32 [n, rot/2], for the rows of this step."""
        key = ("rotary_half", self.theta, self.rotary_dim)
        hit = ctx.shared.get(key)
        if hit is None:
            n = ctx.n_tokens
            cos = ctx.step_alloc((n, self.half), torch.float32)
            sin = ctx.step_alloc((n, self.half), torch.float32)
            ops.rope_table(ctx.batch.positions[:n], self.inv_freq(), cos, sin)
            hit = ctx.shared[key] = (cos, sin)
        return hit

    def rotate(self, ctx, q, k):
        """In place on q [n, heads*head_dim] and k [n, kv_heads*head_dim]."""
        cos, sin = self.prepare(ctx)
        for t in (q, k):
            if t is None:
                continue
            heads = t.shape[1] // self.head_dim
            ops.rope_kv_write(t, t, None, None, cos, sin, self.half, None, None, None, None, None, 0,
                              heads, 0, self.head_dim, False, self.runtime.status)


register_part("position", "rotary_half", RotaryHalf)
