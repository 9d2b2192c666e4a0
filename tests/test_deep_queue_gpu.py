"""A deep model's mixed step with every launch queued ahead of the device.

When the device lags behind the host (a long kernel ahead of the step stands in for that), hundreds of launches
sit in the queue at once and every kernel that may start before its predecessor has ended does so.  The step
must complete, and give the logits of the same step run with the host waiting after every kernel's launch queue
has drained."""
import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(180, method="thread")]

CONFIG = dict(architectures=["MistralForCausalLM"], hidden_size=512, num_hidden_layers=40, num_attention_heads=8,
              num_key_value_heads=2, head_dim=64, intermediate_size=1024, vocab_size=1000, rope_theta=10000.0,
              sliding_window=None, rms_norm_eps=1e-5, tie_word_embeddings=False, hidden_act="silu")


def test_a_mixed_step_of_a_deep_model_queued_ahead_of_the_device():
    from flambeau_b200.config.mistral import MistralConfig
    from flambeau_b200.engine.batch import Entry
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.measure import workloads
    cfg = MistralConfig.from_dict(CONFIG)
    engine = Engine.from_config(cfg, seed=1, options=EngineOptions(
        dtype="bfloat16", cache_tokens=24 * 320 + 2048, max_requests=25, max_step_tokens=600, max_seq_len=2048,
        cuda_graphs=False))
    gen = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, cfg.vocab_size, (24 + 512,), generator=gen).tolist()
    # every page of a pool holds the same random keys and values, put back before each run: what a request sees of
    # its "earlier tokens" then does not depend on which pages the pool hands out, nor on what a run before wrote
    pools = [t for g in engine.cache.groups for c in g.owners for t in (g.k[c], g.v[c])]
    protos = [torch.randn_like(t[:1]) for t in pools]

    def entries():
        for t, proto in zip(pools, protos):
            t.copy_(proto.expand_as(t))
        ids = workloads.seat(engine, [300] * 24 + [513], prefix="q")
        e = [Entry(r, [tokens[i]], [0]) for i, r in enumerate(ids[:-1])]
        e.append(Entry(ids[-1], tokens[24:], [0, 511]))
        return e

    paced = engine.step(entries()).clone()                     # the host is ahead by a few launches at most
    torch.cuda.synchronize()
    results = []
    for _ in range(3):
        batch = entries()
        torch.cuda._sleep(40_000_000)                          # ~20 ms: the whole step is queued behind this
        results.append(engine.step(batch).clone())
    torch.cuda.synchronize()
    engine.runtime.check_status("queued step")
    assert torch.isfinite(paced).all()
    for r in results:
        assert torch.equal(r, paced), "a step's logits depend on how far ahead of the device it was queued"
