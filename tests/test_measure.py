"""The accounting behind the bench line, on the CPU: bytes and flops of a step from the configuration, and the
mapping of launcher calls to kernel classes."""
import pytest

from flambeau_b200.config.mistral import MistralConfig
from flambeau_b200.measure import work
from flambeau_b200.measure.shapes import SHAPES, shape
from flambeau_b200.measure.workloads import classify


def test_shapes_are_valid_configurations():
    for key, s in SHAPES.items():
        cfg = MistralConfig.from_dict(s.config)
        assert cfg.head_dim == 128 and s.context <= cfg.max_position_embeddings
    with pytest.raises(ValueError, match="known"):
        shape("70b")


def test_decode_bytes_of_the_7b_shape():
    """Weights of the layers and the head once (14.22 GB) plus 4,096 live keys of 128 KiB a sequence."""
    cfg = MistralConfig.from_dict(SHAPES["7b"].config)
    s = work.sizes(cfg)
    layer = (s["H"] * (s["qw"] + 2 * s["kvw"]) + s["qw"] * s["H"] + 3 * s["H"] * s["I"] + 2 * s["H"]) * 2
    weights = 32 * layer + s["V"] * s["H"] * 2 + s["H"] * 2
    kv_per_token = 2 * 32 * s["kvw"] * 2
    assert kv_per_token == 128 * 1024
    assert abs(weights - 14.22e9) < 0.01e9
    got = work.decode_step_bytes(weights, kv_per_token, [8192] * 8, s["window"])
    assert got == weights + 8 * 4096 * kv_per_token
    assert work.decode_step_bytes(weights, kv_per_token, [1000], s["window"]) == weights + 1000 * kv_per_token
    assert work.live_keys(8192, 0) == 8192


def test_prefill_flops_of_the_7b_shape():
    cfg = MistralConfig.from_dict(SHAPES["7b"].config)
    flops = work.step_flops(cfg, 32, range(2048), 1)
    assert abs(flops - 29.7e12) < 0.1e12                       # 28.59 linear + 1.10 attention
    assert work.keys_seen(range(10), 4) == 1 + 2 + 3 + 4 * 7
    assert work.keys_seen(range(10), 0) == 55


def test_launcher_calls_fold_into_classes():
    cfg = MistralConfig.from_dict(SHAPES["nemo12b"].config)
    assert classify(cfg, "gemm_tc", (8, 6144, 5120)) == "qkv_proj"
    assert classify(cfg, "gemm_tc", (8, 5120, 4096)) == "o_proj"
    assert classify(cfg, "gemm_tc_gated", (2048, 28672, 5120)) == "gate_up_proj"
    assert classify(cfg, "gemm_tc", (8, 5120, 14336)) == "down_proj"
    assert classify(cfg, "gemm_tc", (8, 131072, 5120)) == "lm_head"
    assert classify(cfg, "add_rms_norm", None) == "add_norm"
    assert classify(cfg, "paged_attention_mma", None) == "attention"
    classes = work.kernel_classes(cfg, 8, [4096] * 8)
    assert classes["attention"]["bytes"] >= 8 * 4096 * 2 * 1024 * 2
    portion = work.kernel_classes(cfg, 2048, [2048])
    assert portion["attention"]["flops"] == 4.0 * work.keys_seen(range(2048), 0) * 4096
    # projections that add to the residual stream themselves read and write it; the norm after them moves less
    assert classify(cfg, "gemm_tc_add", (2048, 5120, 4096)) == "o_proj"
    added = work.kernel_classes(cfg, 2048, [2048], to_stream=True)
    left = work.kernel_classes(cfg, 2048, [2048], to_stream=False)
    H = 5120
    assert left["add_norm"]["bytes"] - added["add_norm"]["bytes"] == 2048 * H * 8
    assert added["o_proj"]["bytes"] - left["o_proj"]["bytes"] == 2048 * H * 4
    assert added["down_proj"]["bytes"] - left["down_proj"]["bytes"] == 2048 * H * 4
