"""Seeded random configurations of the architecture through the engine, against the plain implementation:
head sizes from 16 to 256 in steps of 16, head counts and groups that are no power of two, widths, inner sizes and
vocabularies that are odd multiples, one to three layers, a window or none, tied or untied.  Each runs a mixed
schedule (portions beside decoded tokens, up to four live requests, pages used again) in 32-bit and in bfloat16."""
import random

import pytest

import plain_mistral as pm
import tiny

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    hd = rng.choice(range(16, 257, 16))
    nkv = rng.choice([1, 2, 3, 5])
    group = rng.choice([1, 2, 3, 4, 7])
    while nkv * group * hd > 1536 and group > 1:             # keeps the plain implementation quick
        group -= 1
    return dict(architectures=["MistralForCausalLM"], hidden_size=rng.choice([2, 4, 8]) * rng.randint(5, 40),
                num_hidden_layers=rng.randint(1, 3), num_attention_heads=nkv * group, num_key_value_heads=nkv,
                head_dim=hd, intermediate_size=rng.choice([1, 2, 8]) * rng.randint(3, 60),
                vocab_size=rng.randint(17, 900), rope_theta=rng.choice([1e4, 1e6, 5e5]),
                sliding_window=rng.choice([None, None, 5, 16, 33, 64]), rms_norm_eps=rng.choice([1e-5, 1e-6, 1e-4]),
                tie_word_embeddings=rng.random() < 0.5, hidden_act="silu")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_random_configuration(seed, dtype, tmp_path):
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    cfg = random_config(seed)
    # query/key spread chosen so that scores stay a few units wide whatever the width and the head size
    sharp = (0.2 if dtype == "float32" else 0.1) * (64.0 / cfg["hidden_size"]) ** 0.5 * (16.0 / cfg["head_dim"]) ** 0.25
    folder = tiny.make_folder(tmp_path / "model", cfg, seed=seed, dtype=dtype, sharp=sharp)
    requests = tiny.random_requests(cfg, [3, 37, 90, 21, 70], seed=seed)
    pcfg, W = pm.read_model_folder(folder)
    want = {rid: pm.forward_logits(pcfg, W, toks) for rid, toks in requests.items()}
    sched = tiny.schedule_mixed(requests, seed=seed)
    tokens = sched.max_live_tokens(requests)
    engine = Engine.from_folder(folder, EngineOptions(dtype=dtype, cache_tokens=tokens, max_requests=4,
                                                       max_step_tokens=max(tokens, 128), max_seq_len=max(tokens, 128)))
    replay(engine, sched.lines(), tmp_path / "out")
    engine.cache.check_invariants()
    assert all(g.pool.n_free == g.pool.n_pages for g in engine.cache.groups), "pages lost"
    got = tiny.read_rows(tmp_path / "out", sched, cfg["vocab_size"])
    tiny.compare_rows(got, want, tiny.TOL[dtype], f"seed {seed} {dtype} {cfg}")


def random_mid_config(seed: int) -> dict:
    rng = random.Random(1000 + seed)
    nkv = rng.choice([1, 2, 3, 5])
    return dict(architectures=["MistralForCausalLM"], hidden_size=8 * rng.randint(60, 260), num_hidden_layers=2,
                num_attention_heads=nkv * rng.choice([1, 2, 3, 4]), num_key_value_heads=nkv,
                head_dim=rng.choice([64, 96, 128, 128, 160, 256]), intermediate_size=8 * rng.randint(100, 600),
                vocab_size=rng.randint(2000, 9000), rope_theta=rng.choice([1e4, 1e6]),
                sliding_window=rng.choice([None, 100, 256, 333]), rms_norm_eps=1e-5,
                tie_word_embeddings=rng.random() < 0.5, hidden_act="silu")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [2, 8])
def test_random_mid_size_configuration(seed, dtype, tmp_path):
    """Widths of one to two thousand and prompts of several hundred tokens: the sizes at which the tensor-core
    kernels for portions of prompts run (products with hundreds of rows, attention over a thousand keys), with
    most of each prompt in one step, in long portions of changing size, and mixed."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    cfg = random_mid_config(seed)
    sharp = (0.2 if dtype == "float32" else 0.1) * (64.0 / cfg["hidden_size"]) ** 0.5 * (16.0 / cfg["head_dim"]) ** 0.25
    folder = tiny.make_folder(tmp_path / "model", cfg, seed=seed, dtype=dtype, sharp=sharp)
    rng = random.Random(seed)
    requests = tiny.random_requests(cfg, [rng.randint(300, 1300), rng.randint(40, 700)], seed=seed)
    pcfg, W = pm.read_model_folder(folder)
    want = {rid: pm.forward_logits(pcfg, W, toks) for rid, toks in requests.items()}
    schedules = {"tail": tiny.schedule_tail(requests, 8), "mixed": tiny.schedule_mixed(requests, seed=seed),
                 "portions": tiny.schedule_portions(requests, sizes=(257, 64, 130, 2, 511))}
    for name, sched in schedules.items():
        tokens = sched.max_live_tokens(requests)
        engine = Engine.from_folder(folder, EngineOptions(dtype=dtype, cache_tokens=tokens, max_requests=4,
                                                           max_step_tokens=max(tokens, 128), max_seq_len=max(tokens, 128)))
        replay(engine, sched.lines(), tmp_path / name)
        engine.cache.check_invariants()
        got = tiny.read_rows(tmp_path / name, sched, cfg["vocab_size"])
        tiny.compare_rows(got, want, tiny.TOL[dtype], f"seed {seed} {dtype} {name} {cfg}")
        del engine


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [8, 32, 64])
def test_other_page_sizes(page_size, dtype, tmp_path):
    """The page size is an option of the engine (16 by default, as in the reference): pages of 8, 32 and 64 tokens
    under a window that is no multiple of any of them, with heads of 128 so that the bfloat16 kernels fetch whole
    pages by tensor-map copies, through a mixed schedule with page reuse."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    cfg = dict(architectures=["MistralForCausalLM"], hidden_size=192, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=128, intermediate_size=256, vocab_size=300, rope_theta=1e4,
               sliding_window=70, rms_norm_eps=1e-5, tie_word_embeddings=False, hidden_act="silu")
    sharp = (0.2 if dtype == "float32" else 0.1) * (64.0 / 192) ** 0.5 * (16.0 / 128) ** 0.25
    folder = tiny.make_folder(tmp_path / "model", cfg, seed=page_size, dtype=dtype, sharp=sharp)
    requests = tiny.random_requests(cfg, [150, 37, 200, 21, 90], seed=page_size)
    pcfg, W = pm.read_model_folder(folder)
    want = {rid: pm.forward_logits(pcfg, W, toks) for rid, toks in requests.items()}
    sched = tiny.schedule_mixed(requests, seed=page_size)
    tokens = sched.max_live_tokens(requests)
    engine = Engine.from_folder(folder, EngineOptions(dtype=dtype, page_size=page_size, cache_tokens=tokens,
                                                       max_requests=4, max_step_tokens=256, max_seq_len=256))
    assert engine.cache.page_size == page_size
    replay(engine, sched.lines(), tmp_path / "out")
    engine.runtime.check_status("replay")
    engine.cache.check_invariants()
    assert all(g.pool.n_free == g.pool.n_pages for g in engine.cache.groups), "pages lost"
    got = tiny.read_rows(tmp_path / "out", sched, cfg["vocab_size"])
    tiny.compare_rows(got, want, tiny.TOL[dtype], f"page size {page_size} {dtype}")
