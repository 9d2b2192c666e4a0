"""One layer with the layer sizes of the 7B shape (width 4096, 32 heads / 8 key-value heads of 128, inner 14336,
vocabulary 32000) and one with those of the 12B shape (width 5120 with 32 heads of 128, so heads x head size is not
the width; no window; rope base 1e6; a vocabulary that is no multiple of the product's tiles) against the plain
implementation: the shapes the serving kernels are tuned for (128-wide heads fetched page by page, 128 x 256 product
tiles, split-K slabs), which the tiny configurations do not reach.  The 7B layer's window is shortened to 48 so
that a 150-token request crosses it and gives pages back.  Weights are stored in bfloat16 except the norm weights,
which are stored in float32 and must stay so in the bfloat16 engine."""
import pytest
import torch

import plain_mistral as pm
import tiny

pytestmark = pytest.mark.gpu

CONFIGS = {
    "7b": dict(architectures=["MistralForCausalLM"], hidden_size=4096, num_hidden_layers=1, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32000, rope_theta=10000.0,
               sliding_window=48, rms_norm_eps=1e-5, tie_word_embeddings=False, hidden_act="silu"),
    "12b": dict(architectures=["MistralForCausalLM"], hidden_size=5120, num_hidden_layers=1, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=40010, rope_theta=1e6,
                sliding_window=None, rms_norm_eps=1e-5, tie_word_embeddings=False, hidden_act="silu"),
}


@pytest.fixture(scope="module", params=list(CONFIGS))
def big(request, tmp_path_factory):
    CONFIG = CONFIGS[request.param]
    from flambeau_b200.config.mistral import MistralConfig
    from flambeau_b200.weights.random_init import write_random_model
    folder = tmp_path_factory.mktemp("layer7b")
    write_random_model(folder, MistralConfig.from_dict(CONFIG), seed=5, dtype="bfloat16",
                       float32_names=("layernorm", "model.norm"))
    pcfg, W = pm.read_model_folder(folder)
    requests = tiny.random_requests(CONFIG, [150, 70], seed=2)
    want = {rid: pm.forward_logits(pcfg, W, toks) for rid, toks in requests.items()}
    return dict(folder=folder, requests=requests, want=want, config=CONFIG, name=request.param)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_of_the_7b_shape(big, dtype, tmp_path):
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    reqs = big["requests"]
    engine = Engine.from_folder(big["folder"], EngineOptions(dtype=dtype, cache_tokens=256, max_requests=2,
                                                             max_step_tokens=256, max_seq_len=256))
    if dtype == "bfloat16":
        norm_w = engine.model.layers[0].mixer_norm.weight
        assert norm_w.dtype == torch.float32, "a tensor stored in 32-bit stays so"
        assert engine.model.layers[0].mixer.qkv.weight.dtype == torch.bfloat16
    # whole; then a long portion beside the other request's portions, then single tokens of both
    sched = tiny.Schedule()
    a, b = reqs["r0"], reqs["r1"]
    sched.add([("r0", a[:100], list(range(100)), 0)])
    sched.add([("r0", a[100:130], list(range(30)), 100), ("r1", b[:40], list(range(40)), 0)])
    sched.add([("r0", a[130:132], [0, 1], 130), ("r1", b[40:69], list(range(29)), 40)])
    for i in range(132, 150):
        entries = [("r0", [a[i]], [0], i)]
        if i == 132:
            entries.append(("r1", [b[69]], [0], 69))
        sched.add(entries, end=(["r1"] if i == 132 else []) + (["r0"] if i == 149 else []))
    replay(engine, sched.lines(), tmp_path)
    engine.cache.check_invariants()
    assert not engine.cache.requests
    got = tiny.read_rows(tmp_path, sched, big["config"]["vocab_size"])
    tiny.compare_rows(got, big["want"], tiny.TOL[dtype], f"{big['name']} layer sizes {dtype}")
