"""Each part alone, built from its parameters with random weights and run on a small batch through the same
step context the engine uses, against the plain implementation's function for that part; at sizes that are not
the tiny models' and in both engine dtypes."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_mistral as pm

pytestmark = pytest.mark.gpu


class Bench:
    """A runtime, a cache manager for the given call plans and a step context: what a part needs to run."""

    def __init__(self, dtype, plans=(), cache_tokens=256, max_step_tokens=256):
        from flambeau_b200.engine.runtime import Runtime
        from flambeau_b200.engine.step import Engine, EngineOptions
        self.rt = Runtime("cuda:0", dtype, 16)
        stub = SimpleNamespace(runtime=self.rt, spec=SimpleNamespace(max_positions=None), vocab_size=1000,
                               cache_plans=lambda: list(plans), graph_safe=lambda: False)
        self.engine = Engine(stub, EngineOptions(dtype=dtype, cache_tokens=cache_tokens, max_requests=4,
                                                 max_step_tokens=max_step_tokens, max_seq_len=cache_tokens))

    def begin(self, entries, width):
        from flambeau_b200.engine.batch import Entry
        from flambeau_b200.engine.step import StepContext
        e = self.engine
        entries = [Entry(*x) for x in entries]
        for en in entries:
            if en.request_id not in e.cache.requests:
                e.cache.admit(en.request_id)
            e.cache.reserve(en.request_id, len(en.tokens))
        batch = e.buffers.build(entries, e.cache, 1000)
        self.rt.ws.reset()
        e.step_ws.reset()
        ctx = StepContext(e, batch)
        x = ctx.open_stream(width)
        self._entries = entries
        return ctx, x

    def end(self):
        for en in self._entries:
            self.engine.cache.commit(en.request_id, len(en.tokens))
        torch.cuda.synchronize()
        self.rt.check_status("part")


def bind_random(part, dtype, seed=0):
    from flambeau_b200.weights.random_init import draw
    tensors = {}
    for name, spec in part.tensor_specs().items():
        tensors[name] = draw(spec, seed, name).to(dtype).cuda()
    part.bind(tensors)
    return {k: v.double().cpu() for k, v in tensors.items()}


def rel(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


TOL = {"float32": 5e-6, "bfloat16": 1.5e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from flambeau_b200.parts.norms import RMSNorm
    b = Bench(dtype)
    part = RMSNorm(b.rt, "n.", width=72, eps=3e-4)
    W = bind_random(part, DT[dtype])
    ctx, x = b.begin([("a", [1] * 7, [])], 72)
    x.copy_(torch.randn(7, 72))
    ctx.delta.copy_(torch.randn(7, 72))
    x0, d0 = x.double().cpu(), ctx.delta.double().cpu()
    part.add_norm(ctx, x, ctx.delta, ctx.normed)
    b.end()
    assert rel(x, x0 + d0) < 1e-6
    assert rel(ctx.normed, pm.rms_norm(x0 + d0, W["n.weight"], 3e-4)) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotary_part(dtype):
    from flambeau_b200.parts.positions import RotaryHalf
    b = Bench(dtype)
    part = RotaryHalf(b.rt, "", head_dim=24, theta=5e5, rotary_dim=16)
    ctx, _ = b.begin([("a", [1] * 5, []), ("b", [2] * 3, [])], 8)
    q = torch.randn(8, 3 * 24, device="cuda")
    k = torch.randn(8, 2 * 24, device="cuda")
    q0, k0 = q.double().cpu(), k.double().cpu()
    part.rotate(ctx, q, k)
    b.end()
    pos = torch.tensor([0, 1, 2, 3, 4, 0, 1, 2])
    assert rel(q, pm.rope_split_half(q0.reshape(8, 3, 24), pos, 5e5, 16).reshape(8, -1)) < 5e-6
    assert rel(k, pm.rope_split_half(k0.reshape(8, 2, 24), pos, 5e5, 16).reshape(8, -1)) < 5e-6
    cos, sin = part.prepare(ctx)
    assert cos.shape == (8, 8) and part.prepare(ctx)[0] is cos, "tables are computed once per step"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from flambeau_b200.parts.embedding import LMHead, TokenEmbedding
    b = Bench(dtype)
    emb = TokenEmbedding(b.rt, "e.", vocab=130, width=40)
    head = LMHead(b.rt, "h.", vocab=130, width=40, tied_to="e.weight")
    W = bind_random(emb, DT[dtype])
    head.bind({"h.weight": emb.table})
    assert head.tensor_specs()["h.weight"].alias_of == "e.weight"
    toks = [5, 129, 0, 77]
    ctx, x = b.begin([("a", toks, [])], 40)
    emb.forward(ctx, ctx.batch.token_ids[:4], x)
    h = x.to(DT[dtype])
    logits = torch.empty(4, 130, device="cuda")
    head.forward(ctx, h, logits)
    b.end()
    assert torch.equal(x.double().cpu(), W["e.weight"][toks])
    assert rel(logits, h.double().cpu() @ W["e.weight"].T) < (5e-6 if dtype == "float32" else 1e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [3, 70])
def test_gated_mlp_part(dtype, n):
    from flambeau_b200.parts.feedforward import GatedMLP
    b = Bench(dtype)
    part = GatedMLP(b.rt, "m.", width=56, inner=200, init_std=0.3)
    W = bind_random(part, DT[dtype])
    ctx, _ = b.begin([("a", [1] * n, [])], 56)
    h = torch.randn(n, 56, device="cuda").to(DT[dtype])
    ctx.pending_slabs = 1
    part.forward(ctx, h, ctx.delta)
    b.end()
    got = ctx.delta_slabs[:ctx.pending_slabs].sum(0)
    want = pm.gated_mlp(h.double().cpu(), W["m.gate_proj.weight"], W["m.up_proj.weight"], W["m.down_proj.weight"])
    assert rel(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [0, 9])
def test_attention_part_in_portions(dtype, window):
    """The mixer alone over three steps (a portion, a portion beside another request, single tokens) must give
    what the plain attention block gives on the whole sequences."""
    from flambeau_b200.cache.manager import CallPlan
    from flambeau_b200.parts.attention import PagedAttention
    from flambeau_b200.parts.spec import PartSpec
    width, nh, nkv, hd = 40, 6, 2, 16
    b = None
    part = PagedAttention(None, "a.", width=width, num_heads=nh, num_kv_heads=nkv, head_dim=hd, window=window,
                          init_std=0.2 if dtype == "float32" else 0.1,
                          position=PartSpec("position", "rotary_half", dict(head_dim=hd, theta=1e4)))
    b = Bench(dtype, plans=[CallPlan(kv=part.cache_requirement())])
    part = PagedAttention(b.rt, "a.", width=width, num_heads=nh, num_kv_heads=nkv, head_dim=hd, window=window,
                          init_std=0.2 if dtype == "float32" else 0.1,
                          position=PartSpec("position", "rotary_half", dict(head_dim=hd, theta=1e4)))
    W = bind_random(part, DT[dtype])
    g = torch.Generator().manual_seed(2)
    H = {"a": torch.randn(30, width, generator=g).to(DT[dtype]), "b": torch.randn(21, width, generator=g).to(DT[dtype])}
    steps = [[("a", 0, 17)], [("a", 17, 11), ("b", 0, 20)], [("a", 28, 1), ("b", 20, 1)], [("a", 29, 1)]]
    got = {k: torch.zeros(len(v), width, dtype=torch.float64) for k, v in H.items()}
    for step in steps:
        ctx, _ = b.begin([(rid, [1] * k, []) for rid, _, k in step], width)
        h = torch.cat([H[rid][s:s + k] for rid, s, k in step]).cuda()
        ctx.pending_slabs = 1
        part.forward(ctx, h, ctx.delta, 0)
        b.end()
        out = ctx.delta_slabs[:ctx.pending_slabs].sum(0).double().cpu()
        row = 0
        for rid, s, k in step:
            got[rid][s:s + k] = out[row:row + k]
            row += k
    c = dict(nh=nh, nkv=nkv, hd=hd, theta=1e4, window=window, eps=1.0)
    for rid, h in H.items():
        T = len(h)
        hd_ = h.double()
        q = pm.rope_split_half((hd_ @ W["a.q_proj.weight"].T).reshape(T, nh, hd), torch.arange(T), 1e4)
        k = pm.rope_split_half((hd_ @ W["a.k_proj.weight"].T).reshape(T, nkv, hd), torch.arange(T), 1e4)
        v = (hd_ @ W["a.v_proj.weight"].T).reshape(T, nkv, hd)
        a = pm.attention_causal_window(q, k, v, torch.arange(T), window, 1 / math.sqrt(hd))
        want = a.reshape(T, nh * hd) @ W["a.o_proj.weight"].T
        assert rel(got[rid], want) < TOL[dtype], rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pre_norm_block(dtype):
    from flambeau_b200.cache.manager import CallPlan
    from flambeau_b200.parts.base import KVRequirement
    from flambeau_b200.parts.block import PreNormBlock, ResidualStream
    from flambeau_b200.parts.spec import PartSpec
    width, nh, nkv, hd, inner, eps = 48, 4, 1, 8, 100, 1e-5
    b = Bench(dtype, plans=[CallPlan(kv=KVRequirement(nkv, hd, 0))])
    norm = lambda p: PartSpec("norm", "rmsnorm", dict(width=width, eps=eps), p)
    block = PreNormBlock(b.rt, "L.", mixer=PartSpec("mixer", "attention", dict(
        width=width, num_heads=nh, num_kv_heads=nkv, head_dim=hd, init_std=0.1,
        position=PartSpec("position", "rotary_half", dict(head_dim=hd, theta=1e4))), "L.self_attn."),
        feed_forward=PartSpec("feed_forward", "gated_mlp", dict(width=width, inner=inner, init_std=0.1), "L.mlp."),
        mixer_norm=norm("L.input_layernorm."), feed_forward_norm=norm("L.post_attention_layernorm."))
    W = bind_random(block, DT[dtype])
    T = 19
    ctx, x = b.begin([("a", [1] * T, [])], width)
    x0 = torch.randn(T, width)
    x.copy_(x0)
    stream = ResidualStream(x)
    block.forward(ctx, stream, 0)
    b.end()
    got = x.double().cpu() + ctx.delta_slabs[:stream.pending_slabs].sum(0).double().cpu()   # the last add is pending
    Wm = {k.replace("L.", "model.layers.0."): v for k, v in W.items()}
    c = dict(nh=nh, nkv=nkv, hd=hd, theta=1e4, window=0, eps=eps)
    want = pm.decoder_block(x0.double(), Wm, 0, c, torch.arange(T))
    assert rel(got, want) < TOL[dtype]


def test_pre_norm_block_whose_products_add_to_the_stream():
    """A portion of hundreds of rows in bfloat16: the output projection and the down projection add their results
    to the stream in their own epilogues (nothing is left pending for the next norm), and the block is the plain
    computation's all the same."""
    from flambeau_b200.cache.manager import CallPlan
    from flambeau_b200.parts.base import KVRequirement
    from flambeau_b200.parts.block import PreNormBlock, ResidualStream
    from flambeau_b200.parts.spec import PartSpec
    dtype = "bfloat16"
    width, nh, nkv, hd, inner, eps = 72, 3, 1, 16, 64, 1e-5    # K of 64 at most: no split of K is worth its slab
    T = 333
    b = Bench(dtype, plans=[CallPlan(kv=KVRequirement(nkv, hd, 0))], cache_tokens=512, max_step_tokens=512)
    norm = lambda p: PartSpec("norm", "rmsnorm", dict(width=width, eps=eps), p)
    block = PreNormBlock(b.rt, "L.", mixer=PartSpec("mixer", "attention", dict(
        width=width, num_heads=nh, num_kv_heads=nkv, head_dim=hd, init_std=0.1,
        position=PartSpec("position", "rotary_half", dict(head_dim=hd, theta=1e4))), "L.self_attn."),
        feed_forward=PartSpec("feed_forward", "gated_mlp", dict(width=width, inner=inner, init_std=0.1), "L.mlp."),
        mixer_norm=norm("L.input_layernorm."), feed_forward_norm=norm("L.post_attention_layernorm."))
    W = bind_random(block, DT[dtype])
    ctx, x = b.begin([("a", [1] * T, [])], width)
    x0 = torch.randn(T, width)
    x.copy_(x0)
    stream = ResidualStream(x)
    block.forward(ctx, stream, 0)
    b.end()
    assert stream.pending_slabs == 0, "the down projection left its result for the norm to add"
    Wm = {k.replace("L.", "model.layers.0."): v for k, v in W.items()}
    c = dict(nh=nh, nkv=nkv, hd=hd, theta=1e4, window=0, eps=eps)
    want = pm.decoder_block(x0.double(), Wm, 0, c, torch.arange(T))
    assert rel(x, want) < TOL[dtype]
