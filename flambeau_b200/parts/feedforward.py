"""Gated dense feed-forward (SiLU-gated in the architecture built here)."""
from __future__ import annotations

import os

import torch

from ..kernels import ops
from .base import FeedForward, TensorSpec
from .linear import Linear, interleave_rows
from .spec import register_part


class GatedMLP(FeedForward):
    """d = (act(h Wg^T) * (h Wu^T)) Wd^T, no bias, no routing
    (crates/forward/src/core/composites/dense_ffn.rs:116-186; act = SiLU
    there).  Gate and up weights are stacked at load, row by row alternately,
    so one product yields both and its epilogue can apply the activation to
    neighbouring outputs.  `activation` names one of the kernels' gate
    activations (kernels.ops.ACTIVATIONS)."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, inner: int, activation: str = "silu",
                 init_std: float = 0.02):
        super().__init__(runtime, prefix)
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"gated feed-forward: activation '{activation}' is not implemented "
                             f"({', '.join(sorted(ops.ACTIVATIONS))})")
        self.activation = activation
        self.width, self.inner, self.init_std = int(width), int(inner), init_std
        self.gate_up = self.down = None

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        return {
            p + "gate_proj.weight": TensorSpec((self.inner, self.width), init=init),
            p + "up_proj.weight": TensorSpec((self.inner, self.width), init=init),
            p + "down_proj.weight": TensorSpec((self.width, self.inner), init=init),
        }

    def own_bind(self, tensors):
        p = self.prefix
        self.gate_up = Linear(interleave_rows(tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]))
        self.down = Linear(tensors[p + "down_proj.weight"])
        # Few rows (decoding): when the stacked matrix has at least as many 128-row tiles as the device has SMs,
        # one CTA per tile streams its rows over the whole of K and applies the activation in its epilogue; that
        # many CTAs draw the full memory bandwidth, and the separate activation kernel and the float32 shares it
        # would add are saved (measured on the 7B shape: 1 % of a step at 8 rows, 3 % at 64; a single row is no
        # faster that way and keeps the split).  Narrower matrices keep the split of K, which is what fills the
        # device for them.
        sms = torch.cuda.get_device_properties(self.gate_up.weight.device).multi_processor_count \
            if self.gate_up.weight.is_cuda else 0
        want = os.environ.get("FLAMBEAU_FFN_DECODE_EPILOGUE")
        self.decode_epilogue = (2 * self.inner // 128 >= sms > 0) if want is None else want != "0"

    def own_weights(self):
        return [self.gate_up.weight, self.down.weight]

    def forward(self, ctx, h, out):
        n = ctx.n_tokens
        with ctx.ws.scope():
            a = ctx.ws.alloc((n, self.inner), self.runtime.dtype)
            fused = ops.tc_supported(h, self.gate_up.weight, a)
            if n <= 64 and not (fused and self.decode_epilogue and n >= 2):
                # few rows: float32 split-K shares, added by the activation kernel
                gu = ctx.ws.alloc((ctx.max_slabs, n, 2 * self.inner), torch.float32)
                parts = self.gate_up.slabs(ctx, h, gu)
                ops.gate_mul(gu[0], a, n_partials=parts, partial_stride=gu.stride(0), activation=self.activation)
            elif fused:
                ops.gemm_tc_gated(h, self.gate_up.weight, a, self.runtime.status, self.activation)   # in the epilogue
            else:
                gu = ctx.ws.alloc((n, 2 * self.inner), self.runtime.dtype)
                self.gate_up(ctx, h, gu)
                ops.gate_mul(gu, a, activation=self.activation)
            ctx.to_stream(self.down, a)


register_part("feed_forward", "gated_mlp", GatedMLP)
