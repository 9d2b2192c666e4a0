"""Generality of the parts framework, shown with toy parts that are defined here and never become a model:
a mixer with state of its own (no keys or values), a feed-forward that routes each token to two of four experts,
a position encoding with a rotate() of its own, a query/key norm of the "1 + w" kind hooked into the attention
mixer, a feed-forward gated by another activation, a run order that names a layer twice and lets a call read
another call's cache.  They are registered, built, loaded from a
random model folder and stepped through the engine (whole, in portions, mixed with page reuse, decoded one by
one) without a change to the framework's files, and compared with a plain computation written here."""
import json
import math
from dataclasses import asdict, dataclass

import pytest
import torch

import plain_mistral as pm
import tiny

pytestmark = pytest.mark.gpu


# ---- toy parts ---------------------------------------------------------------------------------------------------

def toy_parts():
    from flambeau_b200.parts.base import FeedForward, Mixer, PositionEncoding, StateRequirement, TensorSpec

    class DecayMixer(Mixer):
        """s_t = a * s_{t-1} + (1 - a) * h_t, out_t = s_t * w: a running average per request, kept in the
        request's state slot between steps.  Tokens of a request must be taken in order."""

        def __init__(self, runtime=None, prefix="", *, width: int, decay: float):
            super().__init__(runtime, prefix)
            self.width, self.decay = width, decay
            self.w = None

        def own_tensor_specs(self):
            return {self.prefix + "w": TensorSpec((self.width,), init=("one_plus_normal", 0.1))}

        def own_bind(self, tensors):
            self.w = tensors[self.prefix + "w"]

        def state_requirement(self):
            return StateRequirement((self.width,), "float32")

        def forward(self, ctx, h, out, call):
            state = ctx.cache(call).state                       # [slots, width] float32
            b = ctx.batch
            for start, length, slot in zip(b.seq_q_start, b.seq_q_len, b.seq_slot):
                s = state[slot]
                for t in range(start, start + length):
                    s = self.decay * s + (1.0 - self.decay) * h[t].float()
                    out[t] = s * self.w.float()
                state[slot] = s

    class ShiftedRotary(PositionEncoding):
        """Rotary pairs (2i, 2i+1) (interleaved, not split-half) with positions shifted by a constant: has its
        own rotate(), so the attention mixer takes its general path."""

        def __init__(self, runtime=None, prefix="", *, head_dim: int, theta: float, shift: int):
            super().__init__(runtime, prefix)
            self.head_dim, self.theta, self.shift = head_dim, theta, shift

        def rotate(self, ctx, q, k):
            n = ctx.n_tokens
            pos = ctx.batch.positions[:n].double() + self.shift
            i = torch.arange(self.head_dim // 2, device=q.device, dtype=torch.float64)
            ang = pos[:, None] * torch.pow(torch.tensor(self.theta, dtype=torch.float64, device=q.device),
                                           -2.0 * i / self.head_dim)[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            for t in (q, k):
                if t is None:
                    continue
                x = t.reshape(n, -1, self.head_dim).double()
                even, odd = x[..., 0::2].clone(), x[..., 1::2].clone()
                x[..., 0::2] = even * c - odd * s
                x[..., 1::2] = even * s + odd * c
                t.copy_(x.reshape(n, -1).to(t.dtype))

    class RoutedFeedForward(FeedForward):
        """Each token goes to the two experts with the largest router logits; an expert's weight is its logit's
        lead over the third-largest over (1 + the sum of both leads), so it falls to zero as the expert leaves the top two and the
        output is continuous in the input.  Experts are relu(h Up^T) Down^T.  Router logits in float32."""

        def __init__(self, runtime=None, prefix="", *, width: int, inner: int, experts: int):
            super().__init__(runtime, prefix)
            self.width, self.inner, self.experts = width, inner, experts
            self.router = self.up = self.down = None

        def own_tensor_specs(self):
            p, E = self.prefix, self.experts
            return {p + "router": TensorSpec((E, self.width), init=("normal", 0.3)),
                    p + "up": TensorSpec((E, self.inner, self.width), init=("normal", 0.2)),
                    p + "down": TensorSpec((E, self.width, self.inner), init=("normal", 0.2))}

        def own_bind(self, tensors):
            p = self.prefix
            self.router, self.up, self.down = tensors[p + "router"], tensors[p + "up"], tensors[p + "down"]

        def forward(self, ctx, h, out):
            n = ctx.n_tokens
            x = h[:n].float()
            weights = routing_weights(x @ self.router.float().T)
            out[:n].zero_()
            for e in range(self.experts):
                rows = (weights[:, e] > 0).nonzero().flatten()             # only the tokens routed here
                if rows.numel():
                    a = torch.relu(x[rows] @ self.up[e].float().T)
                    out[rows] += weights[rows, e:e + 1] * (a @ self.down[e].float().T)

    return DecayMixer, ShiftedRotary, RoutedFeedForward


def routing_weights(logits):
    """[n, E] router logits -> [n, E] weights, zero outside each row's top two."""
    third = logits.topk(3, dim=-1).values[:, 2:3]
    lead = (logits - third).clamp_min(0)
    return lead / (lead.sum(-1, keepdim=True) + 1.0)          # + 1: small leads give small weights, not a 0/0


@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int = 48
    heads: int = 4
    kv_heads: int = 2
    head_dim: int = 8
    inner: int = 56
    vocab_size: int = 97
    eps: float = 1e-5
    theta: float = 100.0
    window: int = 12
    decay: float = 0.8
    experts: int = 4
    expert_inner: int = 20
    attn_std: float = 0.3            # spread of the query/key projections (see SHARP in test_replay_gpu.py)
    architecture = "ToyForCausalLM"

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: v for k, v in raw.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return {**asdict(self), "architectures": ["ToyForCausalLM"]}


# run order: attention (rotary split-half, window) | decay mixer | decay mixer again (same weights, its own
# state) | attention with the toy position encoding, full context | a call of layer 0 again that reads the cache
# of the first call instead of writing one | attention without any rotation, whose positions act through a per-head
# penalty on distance added to the scores
ORDER = [(0, None), (1, None), (1, None), (2, None), (0, 0), (3, None)]


def toy_slopes(cfg):
    """Per query head: 0 for the first (it sees all keys alike), then steeper and steeper."""
    return [0.0 if h == 0 else 2.0 ** (-3.0 * h / cfg.heads) for h in range(cfg.heads)]


def toy_spec(cfg: ToyConfig):
    from flambeau_b200.parts.spec import LayerCall, ModelSpec, PartSpec
    H = cfg.hidden_size

    def norm(prefix):
        return PartSpec("norm", "rmsnorm", dict(width=H, eps=cfg.eps), prefix)

    def ffn(prefix, activation="silu"):
        return PartSpec("feed_forward", "gated_mlp", dict(width=H, inner=cfg.inner, activation=activation), prefix)

    def routed(prefix):
        return PartSpec("feed_forward", "toy_routed", dict(width=H, inner=cfg.expert_inner, experts=cfg.experts), prefix)

    def block(i, mixer):
        p = f"layers.{i}."
        feed_forward = routed(p + "ffn.") if i == 1 else ffn(p + "ffn.", "gelu_tanh" if i == 2 else "silu")
        return PartSpec("block", "pre_norm", dict(mixer=mixer, feed_forward=feed_forward,
                                                  mixer_norm=norm(p + "norm1."), feed_forward_norm=norm(p + "norm2.")), p)

    attn0 = PartSpec("mixer", "attention", dict(
        width=H, num_heads=cfg.heads, num_kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, window=cfg.window,
        init_std=cfg.attn_std, position=PartSpec("position", "rotary_half", dict(head_dim=cfg.head_dim, theta=cfg.theta))),
        "layers.0.attn.")
    decay = PartSpec("mixer", "toy_decay", dict(width=H, decay=cfg.decay), "layers.1.mix.")
    attn2 = PartSpec("mixer", "attention", dict(
        width=H, num_heads=cfg.heads, num_kv_heads=cfg.heads, head_dim=cfg.head_dim, window=0, init_std=cfg.attn_std,
        position=PartSpec("position", "toy_shifted_rotary", dict(head_dim=cfg.head_dim, theta=cfg.theta, shift=5)),
        # a norm over every head of q and k before the rotation, stored as w with 1 + w applied
        qk_norm=PartSpec("norm", "rmsnorm", dict(width=cfg.head_dim, eps=cfg.eps, weight_offset=1.0,
                                                 init=("normal", 0.2)))),
        "layers.2.attn.")
    attn3 = PartSpec("mixer", "attention", dict(
        width=H, num_heads=cfg.heads, num_kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, window=cfg.window,
        init_std=cfg.attn_std, position=None, distance_slopes=toy_slopes(cfg)), "layers.3.attn.")
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab=cfg.vocab_size, width=H, init_std=0.5), "embed."),
        layers=[block(0, attn0), block(1, decay), block(2, attn2), block(3, attn3)],
        order=[LayerCall(l, c) for l, c in ORDER],
        final_norm=norm("final_norm."),
        head=PartSpec("head", "lm_head", dict(vocab=cfg.vocab_size, width=H, init_std=0.1), "head."))


def plain_toy_logits(cfg: ToyConfig, W, tokens):
    """The same model, whole sequence, float64, no cache, no engine code."""
    W = {k: v.double() for k, v in W.items()}
    T = len(tokens)
    pos = torch.arange(T)
    x = pm.embedding(W["embed.weight"], tokens)
    kv = {}
    for c, (layer, cache_from) in enumerate(ORDER):
        p = f"layers.{layer}."
        h = pm.rms_norm(x, W[p + "norm1.weight"], cfg.eps)
        if layer == 1:
            s = torch.zeros(cfg.hidden_size, dtype=torch.float64)
            out = torch.zeros_like(h)
            for t in range(T):
                s = cfg.decay * s + (1 - cfg.decay) * h[t]
                out[t] = s * W[p + "mix.w"]
            x = x + out
        else:
            nh = cfg.heads
            nkv = cfg.heads if layer == 2 else cfg.kv_heads
            a = p + "attn."
            q = (h @ W[a + "q_proj.weight"].T).reshape(T, nh, cfg.head_dim)
            k = (h @ W[a + "k_proj.weight"].T).reshape(T, nkv, cfg.head_dim)
            v = (h @ W[a + "v_proj.weight"].T).reshape(T, nkv, cfg.head_dim)
            if layer == 0:
                q, k = pm.rope_split_half(q, pos, cfg.theta), pm.rope_split_half(k, pos, cfg.theta)
            elif layer == 2:
                q = pm.rms_norm(q, 1.0 + W[a + "q_norm.weight"], cfg.eps)
                k = pm.rms_norm(k, 1.0 + W[a + "k_norm.weight"], cfg.eps)

                def interleaved(t):
                    i = torch.arange(cfg.head_dim // 2, dtype=torch.float64)
                    ang = (pos.double() + 5)[:, None] * (cfg.theta ** (-2.0 * i / cfg.head_dim))[None, :]
                    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                    o = t.clone()
                    o[..., 0::2] = t[..., 0::2] * cs - t[..., 1::2] * sn
                    o[..., 1::2] = t[..., 0::2] * sn + t[..., 1::2] * cs
                    return o
                q, k = interleaved(q), interleaved(k)
            if cache_from is None:
                kv[c] = (k, v)
            else:
                k, v = kv[cache_from]
            window = 0 if layer == 2 else cfg.window
            if layer == 3:                              # no rotation: slope * (key position - query position) on the scores
                att = torch.zeros(T, nh, cfg.head_dim, dtype=torch.float64)
                slopes = toy_slopes(cfg)
                for t in range(T):
                    t0 = max(0, t - window + 1)
                    for hh in range(nh):
                        sc = (k[t0:t + 1, hh // (nh // nkv)] @ q[t, hh]) / math.sqrt(cfg.head_dim) \
                            + slopes[hh] * (torch.arange(t0, t + 1, dtype=torch.float64) - t)
                        att[t, hh] = torch.softmax(sc, dim=0) @ v[t0:t + 1, hh // (nh // nkv)]
            else:
                att = pm.attention_causal_window(q, k, v, pos, window, 1.0 / math.sqrt(cfg.head_dim))
            x = x + att.reshape(T, nh * cfg.head_dim) @ W[a + "o_proj.weight"].T
        h = pm.rms_norm(x, W[p + "norm2.weight"], cfg.eps)
        if layer == 1:
            weights = routing_weights(h @ W[p + "ffn.router"].T)
            for e in range(cfg.experts):
                x = x + weights[:, e:e + 1] * (torch.relu(h @ W[p + "ffn.up"][e].T) @ W[p + "ffn.down"][e].T)
        elif layer == 2:
            g, u = h @ W[p + "ffn.gate_proj.weight"].T, h @ W[p + "ffn.up_proj.weight"].T
            act = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
            x = x + (act * u) @ W[p + "ffn.down_proj.weight"].T
        else:
            x = x + pm.gated_mlp(h, W[p + "ffn.gate_proj.weight"], W[p + "ffn.up_proj.weight"],
                                 W[p + "ffn.down_proj.weight"])
    return pm.rms_norm(x, W["final_norm.weight"], cfg.eps) @ W["head.weight"].T


@pytest.fixture(scope="module")
def registered():
    from flambeau_b200.config.registry import register_architecture, unregister_architecture
    from flambeau_b200.parts.spec import register_part, unregister_part
    DecayMixer, ShiftedRotary, RoutedFeedForward = toy_parts()
    register_part("mixer", "toy_decay", DecayMixer)
    register_part("feed_forward", "toy_routed", RoutedFeedForward)
    register_part("position", "toy_shifted_rotary", ShiftedRotary)
    register_architecture("ToyForCausalLM", ToyConfig, toy_spec)
    yield
    unregister_architecture("ToyForCausalLM")
    unregister_part("mixer", "toy_decay")
    unregister_part("feed_forward", "toy_routed")
    unregister_part("position", "toy_shifted_rotary")


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def toy(request, registered, tmp_path_factory):
    from flambeau_b200.weights.random_init import write_random_model
    cfg = ToyConfig(attn_std=0.3 if request.param == "float32" else 0.15)
    folder = tmp_path_factory.mktemp("toy" + request.param)
    write_random_model(folder, cfg, seed=7, dtype=request.param)
    W = pm.read_safetensors(folder / "model.safetensors")
    requests = tiny.random_requests({"vocab_size": cfg.vocab_size}, [9, 30, 41, 17, 26], seed=3)
    want = {rid: plain_toy_logits(cfg, W, toks) for rid, toks in requests.items()}
    return dict(cfg=cfg, folder=folder, dtype=request.param, requests=requests, want=want)


def test_the_cache_manager_sees_the_toy_model(toy):
    from flambeau_b200.engine.step import Engine, EngineOptions
    e = Engine.from_folder(toy["folder"], EngineOptions(dtype=toy["dtype"], cache_tokens=128, max_requests=3))
    cm = e.cache
    assert cm.n_groups == 2                                    # windowed 2-kv-head group, full 4-kv-head group
    assert set(cm.state) == {1, 2}                             # the two calls of the decay layer: a state each
    assert cm.group_of_call[4] == cm.group_of_call[0] and not cm.view(4, [None, None]).writable
    assert cm.state_bytes_per_request() == 2 * 48 * 4
    assert e.model.layers[1].mixer.__class__.__name__ == "DecayMixer"
    assert e.model.layers[1].feed_forward.__class__.__name__ == "RoutedFeedForward"
    assert e.model.layers[0].feed_forward.__class__.__name__ == "GatedMLP"


@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed1", "mixed2"])
def test_toy_model_steps_like_the_plain_computation(toy, schedule, tmp_path):
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    reqs = toy["requests"]
    sched = {"whole": lambda: tiny.schedule_whole(reqs), "tail": lambda: tiny.schedule_tail(reqs, 12),
             "portions": lambda: tiny.schedule_portions(reqs), "mixed1": lambda: tiny.schedule_mixed(reqs, 1, max_live=3),
             "mixed2": lambda: tiny.schedule_mixed(reqs, 2, max_live=3)}[schedule]()
    tokens = sched.max_live_tokens(reqs)
    engine = Engine.from_folder(toy["folder"], EngineOptions(dtype=toy["dtype"], cache_tokens=tokens, max_requests=3,
                                                             max_step_tokens=128, max_seq_len=128))
    replay(engine, sched.lines(), tmp_path)
    engine.cache.check_invariants()
    assert not engine.cache.requests
    got = tiny.read_rows(tmp_path, sched, toy["cfg"].vocab_size)
    tiny.compare_rows(got, toy["want"], tiny.TOL[toy["dtype"]], f"toy {toy['dtype']} {schedule}")
