"""The model shapes that are benchmarked, as data: config.json contents plus the workload's context length.

Sizes are those of the published checkpoints of the architecture; weights are random."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shape:
    key: str
    name: str
    config: dict          # a MistralForCausalLM config.json
    context: int          # tokens each sequence holds when decoding is measured
    note: str = ""


def _mistral(**kw) -> dict:
    base = dict(architectures=["MistralForCausalLM"], rms_norm_eps=1e-5, tie_word_embeddings=False,
                hidden_act="silu")
    base.update(kw)
    return base


SHAPES = {
    "7b": Shape("7b", "Mistral-7B-v0.1 shape", _mistral(
        hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=14336, vocab_size=32000, rope_theta=10000.0, sliding_window=4096,
        max_position_embeddings=32768), context=8192),
    "nemo12b": Shape("nemo12b", "Mistral-Nemo-12B shape", _mistral(
        hidden_size=5120, num_hidden_layers=40, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=14336, vocab_size=131072, rope_theta=1e6, sliding_window=None,
        max_position_embeddings=131072), context=4096,
        note="heads x head size (4096) is not the width (5120)"),
    "small24b": Shape("small24b", "Mistral-Small-24B shape", _mistral(
        hidden_size=5120, num_hidden_layers=40, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=32768, vocab_size=131072, rope_theta=1e8, sliding_window=None,
        max_position_embeddings=32768), context=4096),
}


def shape(key: str) -> Shape:
    try:
        return SHAPES[key]
    except KeyError:
        raise ValueError(f"unknown shape '{key}'; known: {', '.join(SHAPES)}") from None
