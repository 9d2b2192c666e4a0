"""RMSNorm with the residual add fused in front of it."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, TensorSpec
from .spec import register_part


class RMSNorm(Norm):
    """y = v * (w + weight_offset) / sqrt(mean(v^2) + eps) with v = x + delta.  The
    architecture built here uses the plain weight (weight_offset 0,
    crates/kernels-hip/src/kernels/rmsnorm_f16.cu:41-85); weight_offset 1 is
    the "1 + w" form some architectures store.  The sum, the mean and the
    product are float32; the stream x stays float32."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, eps: float, init=("one_plus_normal", 0.02),
                 weight_offset: float = 0.0):
        super().__init__(runtime, prefix)
        self.width, self.eps, self.init = int(width), float(eps), tuple(init)
        self.weight_offset = float(weight_offset)
        self.weight = None

    def own_tensor_specs(self):
        return {self.prefix + "weight": TensorSpec((self.width,), init=self.init)}

    def own_bind(self, tensors):
        self.weight = tensors[self.prefix + "weight"]

    def own_weights(self):
        return [self.weight]

    def add_norm(self, ctx, x, delta, out, rows=None, n_partials: int = 1):
        if n_partials == 0:                  # the stream already holds the sum
            delta = None
        stride = ctx.delta_slabs.stride(0) if n_partials > 1 else 0
        ops.add_rms_norm(x, delta, self.weight, self.eps, out, rows=rows, n_partials=n_partials,
                         n_rows=ctx.n_tokens, partial_stride=stride, weight_offset=self.weight_offset)

    def normalize(self, ctx, x, out):
        ops.add_rms_norm(x, None, self.weight, self.eps, out, n_rows=x.shape[0], weight_offset=self.weight_offset)


register_part("norm", "rmsnorm", RMSNorm)
