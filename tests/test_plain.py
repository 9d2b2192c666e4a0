"""The plain implementation checked against itself: properties that hold whatever the weights are."""
import math

import pytest
import torch

import plain_mistral as pm
import tiny
from flambeau_b200.config.mistral import MistralConfig
from flambeau_b200.weights.random_init import write_random_model


@pytest.fixture(scope="module", params=["A", "B"])
def model(request, tmp_path_factory):
    folder = tiny.make_folder(tmp_path_factory.mktemp("plain" + request.param), tiny.CONFIGS[request.param],
                              seed=3, dtype="float32")
    return pm.read_model_folder(folder)


def test_causal_prefix_property(model):
    cfg, W = model
    toks = tiny.random_requests(cfg, [30], seed=1)["r0"]
    full = pm.forward_logits(cfg, W, toks)
    short = pm.forward_logits(cfg, W, toks[:17])
    assert torch.allclose(full[:17], short, atol=1e-12)


def test_window_limits_what_a_query_sees():
    T, hd = 12, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(T, 2, hd, generator=g, dtype=torch.float64) for _ in range(3))
    pos = torch.arange(T)
    full = pm.attention_causal_window(q, k, v, pos, 0, 0.3)
    w4 = pm.attention_causal_window(q, k, v, pos, 4, 0.3)
    assert torch.allclose(full[:4], w4[:4])                      # the first W queries see everything so far
    assert not torch.allclose(full[6], w4[6])
    k2, v2 = k.clone(), v.clone()
    k2[:5], v2[:5] = 7.0, -3.0                                   # keys 0..4 are outside the window of query 8
    assert torch.allclose(pm.attention_causal_window(q, k2, v2, pos, 4, 0.3)[8], w4[8])
    w1 = pm.attention_causal_window(q, k, v, pos, 1, 0.3)        # a window of one sees only itself
    assert torch.allclose(w1, v.repeat_interleave(1, dim=1))


@pytest.mark.parametrize("window", [0, 1, 5, 40])
def test_the_masked_matrix_form_of_the_attention_equals_the_loop(window):
    g = torch.Generator().manual_seed(window)
    T = 37
    q = torch.randn(T, 6, 8, generator=g, dtype=torch.float64)
    k, v = (torch.randn(T, 3, 8, generator=g, dtype=torch.float64) for _ in range(2))
    pos = torch.arange(T)
    loop = pm.attention_causal_window(q, k, v, pos, window, 0.35)
    dense = pm.attention_causal_window_dense(q, k, v, pos, window, 0.35)
    assert torch.allclose(loop, dense, atol=1e-13, rtol=0)


def test_whole_model_with_the_masked_matrix_form_and_chosen_rows(model):
    cfg, W = model
    toks = tiny.random_requests(cfg, [45], seed=5)["r0"]
    full = pm.forward_logits(cfg, W, toks)
    some = pm.forward_logits(cfg, W, toks, dense=True, rows=[0, 17, 44])
    assert torch.allclose(full[[0, 17, 44]], some, atol=1e-11, rtol=0)


def test_rope_rotates_pairs_and_keeps_norms():
    x = torch.randn(5, 3, 16, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 50, 1000])
    y = pm.rope_split_half(x, pos, 10000.0)
    assert torch.allclose(y[0], x[0])                            # position 0 is the identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    i = 3
    ang = 2 * 10000.0 ** (-2.0 * i / 16)
    a, b = x[2, 1, i], x[2, 1, i + 8]
    assert math.isclose(float(y[2, 1, i]), float(a * math.cos(ang) - b * math.sin(ang)), rel_tol=1e-12)
    assert math.isclose(float(y[2, 1, i + 8]), float(a * math.sin(ang) + b * math.cos(ang)), rel_tol=1e-12)
    # relative property: q.k after rotation depends on the distance only
    q, k = torch.randn(1, 1, 16, dtype=torch.float64), torch.randn(1, 1, 16, dtype=torch.float64)
    d1 = (pm.rope_split_half(q, torch.tensor([7]), 1e4) * pm.rope_split_half(k, torch.tensor([3]), 1e4)).sum()
    d2 = (pm.rope_split_half(q, torch.tensor([104]), 1e4) * pm.rope_split_half(k, torch.tensor([100]), 1e4)).sum()
    assert math.isclose(float(d1), float(d2), rel_tol=1e-9)


def test_rms_norm_and_mlp_formulas():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = pm.rms_norm(x, w, 0.0 + 1e-30)
    assert torch.allclose(y, torch.tensor([[3.0 * 2 / math.sqrt(12.5), 4.0 * 0.5 / math.sqrt(12.5)]], dtype=torch.float64))
    h = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    out = pm.gated_mlp(h, eye, 2 * eye, eye)
    silu = lambda z: z / (1 + math.exp(-z))
    assert torch.allclose(out, torch.tensor([[silu(1.0) * 2.0, silu(-2.0) * -4.0]], dtype=torch.float64))


def test_tied_head_and_greedy(model):
    cfg, W = model
    toks = [1, 2, 3]
    logits = pm.forward_logits(cfg, W, toks)
    assert logits.shape == (3, cfg["vocab_size"])
    assert ("lm_head.weight" in W) == (not cfg.get("tie_word_embeddings", False))
    gen = pm.greedy_generate(cfg, W, toks, 3)
    assert gen[0] == pm.argmax_lowest(logits[-1])
    assert pm.argmax_lowest(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 1


def test_sampling_oracle():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0])
    p = pm.softmax_temperature(logits, 0.5)
    assert math.isclose(float(p.sum()), 1.0) and float(p[0]) > float(p[1])
    assert pm.inverse_cdf_pick(p, 0.0) == 0 and pm.inverse_cdf_pick(p, 0.999999) == 3
    assert pm.filtered_support(p, top_k=2) == [0, 1]
    assert pm.filtered_support(p, top_p=float(p[0]) - 1e-9) == [0]
    assert pm.filtered_support(p, top_p=float(p[0]) + 1e-9) == [0, 1]
    assert pm.filtered_support(p, min_p=float(p[2] / p[0]) + 1e-9) == [0, 1]
    pen = pm.apply_penalties(torch.tensor([2.0, -2.0, 1.0]), [0, 1, 1], repetition=2.0, presence=0.5, frequency=0.25)
    assert torch.allclose(pen, torch.tensor([2.0 / 2 - 0.5 - 0.25, -2.0 * 2 - 0.5 - 0.5, 1.0], dtype=torch.float64))


def test_weights_read_one_at_a_time_give_the_same_logits(tmp_path):
    """The reader that converts a tensor when it is asked for (for models too large for the host in float64) and the
    reader that converts everything at once are the same numbers."""
    import tiny
    folder = tiny.make_folder(tmp_path / "m", tiny.CONFIG_B, seed=1, dtype="bfloat16")
    cfg, eager = pm.read_model_folder(folder)
    _, lazy = pm.read_model_folder(folder, lazy=True)
    assert set(lazy.keys()) == set(eager.keys())
    tokens = [1, 5, 9, 200, 3, 7, 8]
    assert torch.equal(pm.forward_logits(cfg, eager, tokens), pm.forward_logits(cfg, lazy, tokens))
    many = pm.forward_logits_many(cfg, lazy, {"a": tokens, "b": tokens[:3]})
    assert torch.equal(many["a"], pm.forward_logits(cfg, eager, tokens))
    assert torch.equal(many["b"], pm.forward_logits(cfg, eager, tokens[:3]))
