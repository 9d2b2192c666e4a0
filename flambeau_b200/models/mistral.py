"""Mistral dense (MistralForCausalLM): configuration -> ModelSpec.

Every layer is a pre-norm block of grouped-query attention (rotary positions,
optional sliding window) and a SiLU-gated feed-forward, with RMSNorm before
each and a final RMSNorm before the head; tensor names are the checkpoint's.
This is the reference's plain dense decoder path with its optional extras
switched off (crates/forward/README.md:18-39;
crates/forward/src/ctx.rs:351-411).
"""
from __future__ import annotations

from ..config.mistral import ARCHITECTURE, MistralConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, ModelSpec, PartSpec


def build_spec(cfg: MistralConfig, norm_init=("one_plus_normal", 0.02)) -> ModelSpec:
    H = cfg.hidden_size

    def norm(prefix):
        return PartSpec("norm", "rmsnorm", dict(width=H, eps=cfg.rms_norm_eps, init=norm_init), prefix)

    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        position = PartSpec("position", "rotary_half", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta))
        mixer = PartSpec("mixer", "attention", dict(
            width=H, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, window=cfg.sliding_window or 0, position=position), p + "self_attn.")
        ffn = PartSpec("feed_forward", "gated_mlp", dict(width=H, inner=cfg.intermediate_size,
                                                         activation=cfg.hidden_act), p + "mlp.")
        layers.append(PartSpec("block", "pre_norm", dict(
            mixer=mixer, feed_forward=ffn, mixer_norm=norm(p + "input_layernorm."),
            feed_forward_norm=norm(p + "post_attention_layernorm.")), p))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab=cfg.vocab_size, width=H), "model.embed_tokens."),
        layers=layers,
        order=[LayerCall(i) for i in range(cfg.num_hidden_layers)],
        final_norm=norm("model.norm."),
        head=PartSpec("head", "lm_head", dict(vocab=cfg.vocab_size, width=H,
                                              tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None),
                      "lm_head."),
        max_positions=cfg.max_position_embeddings,
    )


register_architecture(ARCHITECTURE, MistralConfig, build_spec, replace=True)
