"""The shapes that bench.py measures, checked for correctness against the plain implementation.

  * The attention geometry of the 7B shape (32 query / 8 key-value heads of 128, pages of 16) under its real window
    of 4,096 keys: a 4,200-token prompt fed in portions of 512, then 8 tokens decoded one by one, so that portions
    and decoded tokens cross the window's edge and the leading pages are given back.  Width, inner size and
    vocabulary are cut down (they are covered at full size by test_large_shape_gpu.py), which keeps the float64
    oracle to a few seconds.
  * The 7B shape itself, all 32 layers at full sizes: three prompts whole, in portions, with their last
    tokens one by one, and mixed (portions of some beside decoded tokens of others in a pool no larger than needed).  In 32-bit the bound is the 1e-4 of every other test; in bfloat16 it is the
    tiny models' 2e-2 scaled by the square root of the depth (tiny.tol_at_depth says why), and the error that is
    reached is printed.
  * Head sizes that are even but no multiple of 8, which take the kernels' scalar forms.
  * Peak device memory while a model is loaded.
"""
import os

import pytest
import torch

import plain_mistral as pm
import tiny

pytestmark = pytest.mark.gpu

WINDOW_GEOMETRY = dict(architectures=["MistralForCausalLM"], hidden_size=1024, num_hidden_layers=1,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=1536,
                       vocab_size=2000, rope_theta=10000.0, sliding_window=4096, rms_norm_eps=1e-5,
                       tie_word_embeddings=False, hidden_act="silu", max_position_embeddings=32768)

# The whole shape: 14.5 GB of weights on disk (removed when the module's tests are through), 29 GB on the device in
# 32-bit, a minute and a half in all; the oracle reads its float64 weights tensor by tensor.
# FLAMBEAU_TEST_7B_LAYERS=8 runs a quarter of it where disk or time is short; so does a temporary folder with less
# than 30 GB free, or a device with less than 60 GB free (the 32-bit engine holds 29 GB of weights).
def _seven_b_layers() -> int:
    asked = os.environ.get("FLAMBEAU_TEST_7B_LAYERS")
    if asked:
        return int(asked)
    import shutil
    import tempfile
    room = shutil.disk_usage(tempfile.gettempdir()).free >= 30 << 30
    if room and torch.cuda.is_available():
        room = torch.cuda.mem_get_info()[0] >= 60 << 30
    return 32 if room else 8


SEVEN_B_LAYERS = _seven_b_layers()
SEVEN_B = dict(architectures=["MistralForCausalLM"], hidden_size=4096, num_hidden_layers=SEVEN_B_LAYERS, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32000, rope_theta=10000.0,
               sliding_window=4096, rms_norm_eps=1e-5, tie_word_embeddings=False, hidden_act="silu",
               max_position_embeddings=32768)
SEVEN_B_LAYERS_OF_SHAPE = 32


@pytest.fixture(scope="module")
def windowed(tmp_path_factory):
    folder = tiny.make_folder(tmp_path_factory.mktemp("window4096"), WINDOW_GEOMETRY, seed=11, dtype="bfloat16",
                              sharp=0.02)
    pcfg, W = pm.read_model_folder(folder)
    toks = tiny.random_requests(WINDOW_GEOMETRY, [4208], seed=6)["r0"]
    # rows that are checked: around the first portion's end, around the window's edge (queries 4095..4097 are the
    # last to see key 0 and the first not to), the last rows of the prompt, and every decoded token
    rows = [0, 1, 511, 512, 2047, 2048, 4094, 4095, 4096, 4097, 4150, 4198, 4199] + list(range(4200, 4208))
    want = pm.forward_logits(pcfg, W, toks, dense=True, rows=rows)
    return dict(folder=folder, tokens=toks, rows=rows, want=want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_in_portions_of_512_across_the_real_window(windowed, dtype, tmp_path):
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    toks, rows = windowed["tokens"], windowed["rows"]
    # pool: the window, a portion, and the pages a portion's first and last tokens share with their neighbours
    engine = Engine.from_folder(windowed["folder"], EngineOptions(dtype=dtype, cache_tokens=4096 + 512 + 128,
                                                                  max_requests=1, max_step_tokens=512,
                                                                  max_seq_len=8192))
    assert engine.cache.table_pages < 8192 // 16, "a table row holds live pages only"
    sched = tiny.Schedule()
    for p in range(0, 4200, 512):
        k = min(512, 4200 - p)
        sched.add([("r0", toks[p:p + k], [r - p for r in rows if p <= r < p + k], p)])
    for p in range(4200, 4208):
        sched.add([("r0", [toks[p]], [0], p)], end=["r0"] if p == 4207 else [])
    replay(engine, sched.lines(), tmp_path)
    engine.runtime.check_status("replay")
    engine.cache.check_invariants()
    assert not engine.cache.requests
    got = tiny.read_rows(tmp_path, sched, WINDOW_GEOMETRY["vocab_size"])
    want = windowed["want"].numpy()
    scale = float(abs(want).max())
    worst = max(float(abs(got[("r0", r)].astype("float64") - want[i]).max()) / scale for i, r in enumerate(rows))
    print(f"[compare] window 4096, portions of 512, {dtype}: worst error {worst:.3e} of the logit scale")
    assert worst <= tiny.TOL[dtype]


@pytest.fixture(scope="module")
def seven_b(tmp_path_factory):
    from flambeau_b200.config.mistral import MistralConfig
    from flambeau_b200.weights.random_init import write_random_model
    import shutil
    folder = tmp_path_factory.mktemp("sevenb")
    try:
        write_random_model(folder, MistralConfig.from_dict(SEVEN_B), seed=3, dtype="bfloat16")
        pcfg, W = pm.read_model_folder(folder, lazy=True)
        reqs = tiny.random_requests(SEVEN_B, [64, 21, 37], seed=4)
        want = pm.forward_logits_many(pcfg, W, reqs, dense=True)
        yield dict(folder=folder, requests=reqs, want=want)
    finally:
        shutil.rmtree(folder, ignore_errors=True)              # gigabytes: not left to pytest's own clean-up


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_7b_shape_at_depth(seven_b, dtype, tmp_path):
    """The 7B shape, all 32 layers at full size (or as many as FLAMBEAU_TEST_7B_LAYERS says)."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    reqs = seven_b["requests"]
    mixed = tiny.schedule_mixed(reqs, seed=5, max_live=3)
    engine = Engine.from_folder(seven_b["folder"], EngineOptions(dtype=dtype, cache_tokens=mixed.max_live_tokens(reqs),
                                                                 max_requests=3, max_step_tokens=128, max_seq_len=128))
    layers = SEVEN_B["num_hidden_layers"]
    tol = tiny.tol_at_depth(dtype, layers)       # float32: 1e-4 at any depth; bfloat16: 2e-2 * sqrt(layers / 3)
    worst = 0.0
    for name, sched in (("whole", tiny.schedule_whole(reqs)), ("portions", tiny.schedule_portions(reqs)),
                        ("tail", tiny.schedule_tail(reqs, 16)), ("mixed", mixed)):
        out = tmp_path / name
        replay(engine, sched.lines(), out)
        engine.runtime.check_status(name)
        got = tiny.read_rows(out, sched, SEVEN_B["vocab_size"])
        worst = max(worst, tiny.compare_rows(got, seven_b["want"], tol,
                                             f"7B shape, {layers} of {SEVEN_B_LAYERS_OF_SHAPE} layers, {dtype}, {name}"))
    print(f"[depth] 7B shape at {layers} layers, {dtype}: worst error {worst:.3e} (bound {tol:.2e})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 20), (3, 3, 18), (4, 1, 36)])
def test_head_sizes_that_are_no_multiple_of_8(nh, nkv, hd, dtype, tmp_path):
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    cfg = dict(architectures=["MistralForCausalLM"], hidden_size=72, num_hidden_layers=2, num_attention_heads=nh,
               num_key_value_heads=nkv, head_dim=hd, intermediate_size=100, vocab_size=211, rope_theta=1e4,
               sliding_window=24, rms_norm_eps=1e-5, tie_word_embeddings=False, hidden_act="silu")
    folder = tiny.make_folder(tmp_path / "model", cfg, seed=hd, dtype=dtype, sharp=0.2 if dtype == "float32" else 0.1)
    requests = tiny.random_requests(cfg, [3, 37, 90, 21], seed=hd)
    pcfg, W = pm.read_model_folder(folder)
    want = {rid: pm.forward_logits(pcfg, W, toks) for rid, toks in requests.items()}
    sched = tiny.schedule_mixed(requests, seed=hd)
    tokens = sched.max_live_tokens(requests)
    engine = Engine.from_folder(folder, EngineOptions(dtype=dtype, cache_tokens=tokens, max_requests=4,
                                                       max_step_tokens=128, max_seq_len=128))
    replay(engine, sched.lines(), tmp_path / "out")
    engine.runtime.check_status("replay")
    engine.cache.check_invariants()
    got = tiny.read_rows(tmp_path / "out", sched, cfg["vocab_size"])
    tiny.compare_rows(got, want, tiny.TOL[dtype], f"head size {hd} {dtype}")


def test_loading_holds_little_more_than_the_weights(seven_b):
    """Query/key/value and gate/up weights are stacked into one buffer each when a part is bound; the model is
    loaded and bound part by part, so only one layer's tensors are on the device twice at any time."""
    from flambeau_b200.engine.runtime import Runtime
    from flambeau_b200.weights.loader import load_model
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    model = load_model(seven_b["folder"], Runtime("cuda:0", "bfloat16"))
    torch.cuda.synchronize()
    held = torch.cuda.memory_allocated() - before
    peak = torch.cuda.max_memory_allocated() - before
    weights = sum(t.numel() * t.element_size() for p in model.parts() for t in _tensors(p))
    print(f"[load] weights {weights / 2**30:.2f} GiB, held {held / 2**30:.2f} GiB, peak {peak / 2**30:.2f} GiB")
    assert peak <= 1.15 * weights + (64 << 20)


def _tensors(part):
    seen = []
    for t in part.own_weights() + ([part.table] if hasattr(part, "table") and part.table is not None else []):
        seen.append(t)
    for c in part.children():
        seen += _tensors(c)
    return seen
