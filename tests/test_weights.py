"""Safetensors reading/writing, the weight loader's one error, and the random-weights mode (CPU)."""
import json

import pytest
import torch

import plain_mistral as pm
import tiny
from flambeau_b200.config.mistral import MistralConfig
from flambeau_b200.weights.loader import WeightError, load_tensors
from flambeau_b200.weights.random_init import model_tensor_specs, write_random_model
from flambeau_b200.weights.safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, write_safetensors


class FakeRuntime:
    """The loader only needs a device and the dtype rule."""
    device = torch.device("cpu")

    def __init__(self, full_precision=False):
        self.full_precision = full_precision

    def weight_dtype(self, stored):
        if self.full_precision or stored in (torch.float32, torch.float64):
            return torch.float32
        return torch.bfloat16


def test_round_trip_and_independent_reader(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "d": torch.tensor(2.5)}
    write_safetensors(tmp_path / "model.safetensors", tensors, metadata={"k": "v"})
    f = SafetensorsFile(tmp_path / "model.safetensors")
    assert sorted(f.names()) == ["a", "b", "c", "d"] and f.metadata == {"k": "v"}
    for n, t in tensors.items():
        assert f.dtype(n) == t.dtype and torch.equal(f.tensor(n), t)
    plain = pm.read_safetensors(tmp_path / "model.safetensors")
    assert torch.equal(plain["b"], tensors["b"].double()) and torch.equal(plain["a"], tensors["a"].double())


def test_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError):
        ModelFiles(tmp_path / "nothing")


@pytest.mark.parametrize("name", ["A", "B"])
def test_random_model_is_seeded_and_complete(tmp_path, name):
    cfg = MistralConfig.from_dict(tiny.CONFIGS[name])
    write_random_model(tmp_path / "m1", cfg, seed=4, dtype="bfloat16")
    write_random_model(tmp_path / "m2", cfg, seed=4, dtype="bfloat16")
    write_random_model(tmp_path / "m3", cfg, seed=5, dtype="float32")
    f1, f2, f3 = (ModelFiles(tmp_path / m) for m in ("m1", "m2", "m3"))
    specs = model_tensor_specs(cfg)
    stored = {n for n, s in specs.items() if s.alias_of is None}
    assert set(f1.names()) == stored
    assert ("lm_head.weight" in stored) == (not cfg.tie_word_embeddings)
    for n in stored:
        assert torch.equal(f1.tensor(n), f2.tensor(n))
        assert f1.dtype(n) == torch.bfloat16 and f3.dtype(n) == torch.float32
        assert tuple(f1.shape(n)) == tuple(specs[n].shape)
    assert not torch.equal(f1.tensor("model.embed_tokens.weight").float(), f3.tensor("model.embed_tokens.weight"))
    w = f3.tensor("model.layers.0.self_attn.q_proj.weight")
    assert abs(float(w.std()) - 0.02) < 0.004
    nw = f3.tensor("model.norm.weight")
    assert abs(float(nw.mean()) - 1.0) < 0.05
    assert json.loads((tmp_path / "m1" / "config.json").read_text())["architectures"] == ["MistralForCausalLM"]
    assert MistralConfig.from_json(tmp_path / "m1") == cfg


def test_loader_keeps_dtypes_by_the_rule(tmp_path):
    cfg = MistralConfig.from_dict(tiny.CONFIG_A)
    write_random_model(tmp_path, cfg, seed=1, dtype="bfloat16", float32_names=("layernorm", "model.norm"))
    specs = model_tensor_specs(cfg)
    t = load_tensors(tmp_path, specs, FakeRuntime())
    assert t["model.layers.0.input_layernorm.weight"].dtype == torch.float32      # stored in 32-bit: stays
    assert t["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    t32 = load_tensors(tmp_path, specs, FakeRuntime(full_precision=True))
    assert all(v.dtype == torch.float32 for v in t32.values())


def test_tied_head_is_the_embedding(tmp_path):
    cfg = MistralConfig.from_dict(tiny.CONFIG_B)
    write_random_model(tmp_path, cfg, seed=1)
    t = load_tensors(tmp_path, model_tensor_specs(cfg), FakeRuntime())
    assert t["lm_head.weight"].data_ptr() == t["model.embed_tokens.weight"].data_ptr()


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    cfg = MistralConfig.from_dict(tiny.CONFIG_A)
    write_random_model(tmp_path, cfg, seed=1)
    f = SafetensorsFile(tmp_path / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    tensors["model.layers.0.mlp.up_proj.weight"] = torch.zeros(128, 64, dtype=torch.int32)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_tensors(tmp_path, model_tensor_specs(cfg), FakeRuntime())
    err = e.value
    assert err.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert len(err.wrong) == 2 and "k_proj" in " ".join(err.wrong) and "up_proj" in " ".join(err.wrong)
    msg = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape or type (2)", "[16, 64]", "[32, 64]"):
        assert needle in msg


def test_linear_weights_stored_in_32_bit_are_kept_and_warned_about(tmp_path):
    """A tensor stored in 32-bit stays so in bfloat16 mode.  For norm weights that is wanted; a linear map kept in
    float32 runs on the FMA kernel, so the loader says so once."""
    import warnings
    cfg = MistralConfig.from_dict(tiny.CONFIGS["A"])
    write_random_model(tmp_path / "f32", cfg, seed=1, dtype="float32")
    write_random_model(tmp_path / "mixed", cfg, seed=1, dtype="bfloat16", float32_names=("layernorm", "model.norm"))
    specs = model_tensor_specs(cfg)
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        got = load_tensors(tmp_path / "f32", specs, FakeRuntime())
    assert all(t.dtype == torch.float32 for t in got.values())
    assert sum("32-bit" in str(w.message) for w in seen) == 1, "one warning, not one per tensor"
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        got = load_tensors(tmp_path / "mixed", specs, FakeRuntime())
    assert not seen, "norm weights in 32-bit are the usual case and need no warning"
    assert got["model.norm.weight"].dtype == torch.float32
    assert got["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16


def test_model_is_bound_part_by_part_and_a_tied_head_is_one_tensor(tmp_path):
    from flambeau_b200.weights.loader import FolderTensors
    cfg = MistralConfig.from_dict(tiny.CONFIGS["B"])                    # tied
    write_random_model(tmp_path / "m", cfg, seed=2, dtype="bfloat16")
    specs = model_tensor_specs(cfg)
    ft = FolderTensors(tmp_path / "m", specs, FakeRuntime())
    emb = ft.fetch(["model.embed_tokens.weight"])["model.embed_tokens.weight"]
    layer = ft.fetch([n for n in specs if n.startswith("model.layers.1.")])
    head = ft.fetch(["lm_head.weight"])["lm_head.weight"]
    ft.close()
    assert head.data_ptr() == emb.data_ptr(), "a tied head is the embedding tensor under a second name"
    assert len(layer) == 9
