"""Token embedding and output head."""
from __future__ import annotations

from ..kernels import ops
from .base import Part, TensorSpec
from .linear import Linear
from .spec import register_part


class TokenEmbedding(Part):
    """x[t,:] = E[token[t],:], no scale (crates/forward/src/core/composites/embed.rs:26-62)."""
    graph_safe = True
    category = "embedding"

    def __init__(self, runtime=None, prefix="", *, vocab: int, width: int, init_std: float = 0.02):
        super().__init__(runtime, prefix)
        self.vocab, self.width, self.init_std = int(vocab), int(width), init_std
        self.table = None

    def own_tensor_specs(self):
        return {self.prefix + "weight": TensorSpec((self.vocab, self.width), init=("normal", self.init_std))}

    def own_bind(self, tensors):
        self.table = tensors[self.prefix + "weight"]

    def own_weights(self):
        return []          # a step reads n rows of the table, not the table

    def forward(self, ctx, token_ids, x):
        ops.embedding(self.table, token_ids, x, self.runtime.status)


class LMHead(Part):
    """logits = h W^T in float32, for the wanted rows only; a tied head reuses
    the embedding table (crates/forward/src/core/composites/output_head.rs:90-132;
    crates/models/qwen35-v2/src/loader.rs:219-223)."""
    graph_safe = True
    category = "head"

    def __init__(self, runtime=None, prefix="", *, vocab: int, width: int, tied_to: str | None = None,
                 init_std: float = 0.02):
        super().__init__(runtime, prefix)
        self.vocab, self.width, self.tied_to, self.init_std = int(vocab), int(width), tied_to, init_std
        self.proj = None

    def own_tensor_specs(self):
        return {self.prefix + "weight": TensorSpec((self.vocab, self.width), init=("normal", self.init_std),
                                                   alias_of=self.tied_to)}

    def own_bind(self, tensors):
        self.proj = Linear(tensors[self.prefix + "weight"])

    def own_weights(self):
        return [self.proj.weight]

    def forward(self, ctx, h_rows, logits):
        self.proj(ctx, h_rows, logits)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
