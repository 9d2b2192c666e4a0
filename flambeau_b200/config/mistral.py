"""MistralConfig: the keys of a MistralForCausalLM config.json, typed.

Field names are the config.json keys.  Requiredness and defaults follow the
reference's dense-decoder metadata reader
(crates/models/qwen35-v2/src/config.rs:55-64: width, layer count, head counts,
feed-forward length and norm eps are required; head size defaults to
width / heads; rope base defaults to 10000).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

from .base import BadValue, ConfigReader, WrongArchitecture, read_config_json

ARCHITECTURE = "MistralForCausalLM"


@dataclass(frozen=True)
class MistralConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    sliding_window: Optional[int] = None      # keys a query sees, itself included; None = all
    tie_word_embeddings: bool = False
    max_position_embeddings: Optional[int] = None
    hidden_act: str = "silu"

    architecture = ARCHITECTURE

    # ---- reading ---------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "MistralConfig":
        r = ConfigReader(raw)
        arch = r.architecture()
        if arch != ARCHITECTURE:
            raise WrongArchitecture(raw.get("architectures"), ARCHITECTURE)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        if heads % kv_heads:
            raise BadValue("num_key_value_heads", kv_heads,
                           f"must divide num_attention_heads = {heads}")
        head_dim = r.integer("head_dim", default=None, minimum=1)
        if head_dim is None:
            if hidden % heads:
                raise BadValue("hidden_size", hidden,
                               f"not a multiple of num_attention_heads = {heads} and no head_dim given")
            head_dim = hidden // heads
        if head_dim % 2:
            raise BadValue("head_dim", head_dim, "rotary pairs need an even head size")
        window = r.integer("sliding_window", default=None, minimum=0)
        if window == 0:
            window = None
        act = r.string("hidden_act", default="silu")
        if act != "silu":
            raise BadValue("hidden_act", act, "the gated feed-forward of this architecture uses 'silu'")
        if raw.get("rope_scaling") is not None:
            raise BadValue("rope_scaling", raw["rope_scaling"], "scaled rotary variants are not supported")
        return cls(
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            vocab_size=r.integer("vocab_size", minimum=1),
            rms_norm_eps=r.number("rms_norm_eps", positive=True),
            rope_theta=r.number("rope_theta", default=10000.0, positive=True),
            sliding_window=window,
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
            max_position_embeddings=r.integer("max_position_embeddings", default=None, minimum=1),
            hidden_act=act,
        )

    @classmethod
    def from_json(cls, folder_or_file) -> "MistralConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    # ---- writing ---------------------------------------------------------
    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [ARCHITECTURE]
        d["model_type"] = "mistral"
        return d
