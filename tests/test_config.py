"""Configuration and registry (CPU)."""
import json

import pytest

import tiny
from flambeau_b200 import models  # noqa: F401
from flambeau_b200.config.base import BadValue, ConfigError, MissingKey, WrongArchitecture
from flambeau_b200.config.mistral import MistralConfig
from flambeau_b200.config.registry import (UnknownArchitecture, known_architectures, load_config,
                                           register_architecture, resolve, unregister_architecture)


def test_reads_every_key_of_both_tiny_configs():
    a = MistralConfig.from_dict(tiny.CONFIG_A)
    b = MistralConfig.from_dict(tiny.CONFIG_B)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 2, 4, 2, 16)
    assert (a.intermediate_size, a.vocab_size, a.rope_theta, a.sliding_window, a.rms_norm_eps) == (128, 256, 1e4, 16, 1e-5)
    assert not a.tie_word_embeddings
    assert (b.hidden_size, b.num_hidden_layers, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 3, 8, 1, 24)
    assert b.sliding_window is None and b.tie_word_embeddings and b.rope_theta == 1e6 and b.rms_norm_eps == 1e-6


def test_defaults():
    raw = dict(architectures=["MistralForCausalLM"], hidden_size=64, num_hidden_layers=1, num_attention_heads=4,
               intermediate_size=8, vocab_size=10, rms_norm_eps=1e-5)
    c = MistralConfig.from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16 and c.rope_theta == 10000.0
    assert c.sliding_window is None and not c.tie_word_embeddings and c.hidden_act == "silu"
    assert MistralConfig.from_dict({**raw, "sliding_window": 0}).sliding_window is None


def test_round_trip(tmp_path):
    c = MistralConfig.from_dict(tiny.CONFIG_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    arch, again = load_config(tmp_path)
    assert arch.name == "MistralForCausalLM" and again == c


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "rms_norm_eps"])
def test_missing_required_key(key):
    raw = dict(tiny.CONFIG_A)
    del raw[key]
    with pytest.raises(MissingKey) as e:
        MistralConfig.from_dict(raw)
    assert key in str(e.value)


def test_wrong_architecture_and_bad_values():
    with pytest.raises(WrongArchitecture):
        MistralConfig.from_dict({**tiny.CONFIG_A, "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(MissingKey):
        MistralConfig.from_dict({k: v for k, v in tiny.CONFIG_A.items() if k != "architectures"})
    for bad in (dict(num_key_value_heads=3), dict(head_dim=15), dict(hidden_act="gelu"),
                dict(rope_scaling={"type": "linear"}), dict(hidden_size="64"), dict(rms_norm_eps=0.0),
                dict(num_hidden_layers=0), dict(tie_word_embeddings="yes")):
        with pytest.raises(BadValue):
            MistralConfig.from_dict({**tiny.CONFIG_A, **bad})
    with pytest.raises(BadValue):      # width not divisible by heads and no head_dim
        MistralConfig.from_dict({**{k: v for k, v in tiny.CONFIG_A.items() if k != "head_dim"}, "hidden_size": 66})


def test_registry_lists_known_names_on_a_miss():
    assert "MistralForCausalLM" in known_architectures()
    with pytest.raises(UnknownArchitecture) as e:
        resolve("GPT2LMHeadModel")
    assert "MistralForCausalLM" in str(e.value)


def test_registry_takes_another_architecture():
    register_architecture("ToyForCausalLM", MistralConfig, lambda cfg: None)
    try:
        assert resolve("ToyForCausalLM").config_class is MistralConfig
        with pytest.raises(ConfigError):
            register_architecture("ToyForCausalLM", MistralConfig, lambda cfg: None)
    finally:
        unregister_architecture("ToyForCausalLM")


def test_config_file_errors(tmp_path):
    with pytest.raises(ConfigError):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(tmp_path)
