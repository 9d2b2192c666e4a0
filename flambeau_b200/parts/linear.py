"""A bias-free linear map y = a W^T with W stored [outputs, inputs]
(crates/forward/src/loader/shard.rs:81-83)."""
from __future__ import annotations

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError("a linear weight is 2-d [outputs, inputs]")
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def __call__(self, ctx, a: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.linear(a, self.weight, out, ctx)
        return out

    def slabs(self, ctx, a: torch.Tensor, slabs: torch.Tensor) -> int:
        """The product as a sum of float32 slabs (split-K shares that the next kernel adds); returns how many."""
        return ops.linear_slabs(a, self.weight, slabs, ctx)

    def add_into(self, ctx, a: torch.Tensor, acc: torch.Tensor) -> bool:
        """acc += a W^T where the product's own epilogue can do the add (see ops.gemm_tc_add); False, with nothing
        done, where it cannot."""
        return ops.gemm_tc_add(a, self.weight, acc, ctx.runtime.status, ctx.max_slabs)


def interleave_rows(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Rows a_0, b_0, a_1, b_1, ...: two maps of one input whose outputs are wanted side by side."""
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError("interleaved weights must share shape and dtype")
    return torch.stack([a, b], dim=1).reshape(2 * a.shape[0], a.shape[1]).contiguous()


def concat_rows(tensors) -> torch.Tensor:
    """Stack weights that share their input so one product serves them all."""
    dts = {t.dtype for t in tensors}
    if len(dts) != 1:
        raise ValueError(f"fused weights must share a dtype, got {dts}")
    return torch.cat(list(tensors), dim=0).contiguous()
