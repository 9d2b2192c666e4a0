"""Plain, slow Mistral-dense implementation used only as the oracle of the tests.

It rests on the formulas of arte-fact/flambeau's dense decoder path (its model
code is Rust + HIP and can be neither imported nor compiled on a CPU-only
Python box, so nothing here was checked against a run of it; every function
cites the file and lines of the reference that give the formula).

Whole sequences, no cache, one function for each part, float64 on the CPU.
Nothing in this file imports the engine: it has its own config and safetensors
reading so that a fault in the product's loader cannot hide in both.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------
# model folder reading (independent of flambeau_b200.weights)
# --------------------------------------------------------------------------

_NP_DTYPES = {"F32": np.float32, "F64": np.float64, "F16": np.float16,
              "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """name -> float64 tensor (integer tensors stay integer)."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[base + lo: base + hi]
        shape = info["shape"]
        dt = info["dtype"]
        if dt == "BF16":
            u16 = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(buf, dtype=_NP_DTYPES[dt])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = torch.from_numpy(arr.reshape(shape).copy())
    return out


class LazyWeights:
    """name -> float64 tensor like read_safetensors, but every tensor is read and converted when it is asked for and
    not kept: for models whose weights in float64 would not fit the host's memory at once."""

    def __init__(self, path):
        self.path = Path(path)
        with open(self.path, "rb") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            self.header = {k: v for k, v in json.loads(f.read(hlen)).items() if k != "__metadata__"}
        self.base = 8 + hlen

    def __contains__(self, name):
        return name in self.header

    def keys(self):
        return self.header.keys()

    def __getitem__(self, name):
        info = self.header[name]
        lo, hi = info["data_offsets"]
        with open(self.path, "rb") as f:
            f.seek(self.base + lo)
            buf = f.read(hi - lo)
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(buf, dtype=_NP_DTYPES[info["dtype"]])
            arr = arr.astype(np.float64) if arr.dtype.kind == "f" else arr.copy()
        return torch.from_numpy(arr.reshape(info["shape"]))


def read_model_folder(folder, lazy: bool = False):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = LazyWeights(folder / "model.safetensors") if lazy else read_safetensors(folder / "model.safetensors")
    return cfg, weights


def _cfg(cfg: dict):
    """The numbers the formulas need, with the defaults the reference gives
    (crates/models/qwen35-v2/src/config.rs:55-64: head_dim defaults to
    hidden/heads, rope base to 10000)."""
    nh = cfg["num_attention_heads"]
    return dict(
        H=cfg["hidden_size"], L=cfg["num_hidden_layers"], nh=nh,
        nkv=cfg.get("num_key_value_heads") or nh,
        hd=cfg.get("head_dim") or cfg["hidden_size"] // nh,
        theta=float(cfg.get("rope_theta", 10000.0)),
        window=int(cfg.get("sliding_window") or 0),
        eps=float(cfg["rms_norm_eps"]),
        tied=bool(cfg.get("tie_word_embeddings", False)),
    )


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embedding(table: torch.Tensor, tokens) -> torch.Tensor:
    """x[t,:] = E[token[t],:], no scale.
    crates/forward/src/core/composites/embed.rs:26-62."""
    idx = torch.as_tensor(tokens, dtype=torch.long)
    if int(idx.max()) >= table.shape[0] or int(idx.min()) < 0:
        raise ValueError("token id outside the vocabulary")
    return table[idx].to(F64)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """ms = sum(x^2)/H; y = x * w / sqrt(ms + eps); plain weight, no 1+w.
    crates/kernels-hip/src/kernels/rmsnorm_f16.cu:41-85;
    crates/model-ops/src/ops/rmsnorm.rs:197-220."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * w / torch.sqrt(ms + eps)


def rope_split_half(x: torch.Tensor, positions: torch.Tensor, theta: float,
                    rot: int | None = None) -> torch.Tensor:
    """x: [T, heads, hd]. For pair i in [0, rot/2): angle = pos * theta^(-2i/rot);
    (x[i], x[i+rot/2]) <- (x[i] cos - x[i+rot/2] sin, x[i] sin + x[i+rot/2] cos).
    crates/kernels-hip/src/kernels/rope_neox_partial_f16.cu:39-52;
    crates/model-ops/src/ops/rope.rs:120-148."""
    T, nheads, hd = x.shape
    rot = hd if rot is None else rot
    half = rot // 2
    i = torch.arange(half, dtype=F64)
    inv = theta ** (-2.0 * i / rot)
    ang = positions.to(F64)[:, None] * inv[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    lo, hi = x[..., :half], x[..., half:rot]
    out = x.clone()
    out[..., :half] = lo * c - hi * s
    out[..., half:rot] = lo * s + hi * c
    return out


def attention_causal_window(q, k, v, positions, window: int, scale: float):
    """q: [T, nh, hd]; k, v: [T, nkv, hd]. Query at position p of q-head g uses
    kv-head g // (nh/nkv) and sees keys t in [max(0, p-W+1), p] (all of [0, p]
    when W == 0); scores scale * q.k, softmax over the visible keys, then the
    weighted sum of v.
    crates/kernels-hip/src/kernels/attention_prefill_f16_paged.cu:69-149;
    crates/model-ops/src/ops/attn_prefill.rs:92-140;
    crates/ops/tests/swa_softcap_parity.rs:130-186."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    out = torch.zeros_like(q)
    pos = [int(p) for p in positions]
    for g in range(nh):
        kvh = g // rep
        scores = scale * (q[:, g, :] @ k[:, kvh, :].T)        # [T, T]
        for a in range(T):
            p = pos[a]
            t0 = max(0, p - window + 1) if window > 0 else 0
            vis = [b for b in range(T) if t0 <= pos[b] <= p]
            s = scores[a, vis]
            w = torch.softmax(s, dim=0)
            out[a, g, :] = w @ v[vis, kvh, :]
    return out


def attention_causal_window_dense(q, k, v, positions, window: int, scale: float):
    """The formula of attention_causal_window with a mask over the whole score matrix instead of a loop over
    queries, for sequences of thousands of tokens (tests/test_plain.py holds the two against each other).
    Keys outside [max(0, p-W+1), p] get a weight of exactly zero."""
    T, nh, hd = q.shape
    rep = nh // k.shape[1]
    pos = positions.to(torch.long)
    seen = pos[None, :] <= pos[:, None]
    if window > 0:
        seen &= pos[None, :] >= (pos[:, None] - window + 1)
    out = torch.zeros_like(q)
    for g in range(nh):
        scores = scale * (q[:, g, :] @ k[:, g // rep, :].T)
        scores = scores.masked_fill(~seen, -math.inf)
        out[:, g, :] = torch.softmax(scores, dim=-1) @ v[:, g // rep, :]
    return out


def gated_mlp(h, w_gate, w_up, w_down):
    """g = h Wg^T, u = h Wu^T, a = g/(1+exp(-g)) * u, d = a Wd^T; no bias.
    crates/forward/src/core/composites/dense_ffn.rs:116-186;
    crates/model-ops/src/ops/activation.rs:107-118."""
    g = h @ w_gate.T
    u = h @ w_up.T
    a = g / (1.0 + torch.exp(-g)) * u
    return a @ w_down.T


def attention_block(x, W, prefix, c, positions, dense: bool = False):
    """h = norm(x); q,k,v = h Wq^T, h Wk^T, h Wv^T (no bias); rope on q and k
    after projection and before use; attention; o = a Wo^T.
    crates/forward/src/core/composites/standard_attn.rs:130-158, 197-286,
    355-399, 1261-1302; scale 1/sqrt(hd) from :418-420."""
    T = x.shape[0]
    h = rms_norm(x, W[prefix + "input_layernorm.weight"], c["eps"])
    q = (h @ W[prefix + "self_attn.q_proj.weight"].T).reshape(T, c["nh"], c["hd"])
    k = (h @ W[prefix + "self_attn.k_proj.weight"].T).reshape(T, c["nkv"], c["hd"])
    v = (h @ W[prefix + "self_attn.v_proj.weight"].T).reshape(T, c["nkv"], c["hd"])
    q = rope_split_half(q, positions, c["theta"])
    k = rope_split_half(k, positions, c["theta"])
    attend = attention_causal_window_dense if dense else attention_causal_window
    a = attend(q, k, v, positions, c["window"], 1.0 / math.sqrt(c["hd"]))
    return a.reshape(T, c["nh"] * c["hd"]) @ W[prefix + "self_attn.o_proj.weight"].T


def decoder_block(x, W, layer: int, c, positions, dense: bool = False):
    """x = x + attention(norm(x)); x = x + mlp(norm(x)).
    crates/models/qwen35-v2/src/model.rs:25-42;
    crates/forward/src/core/composites/residual_add.rs:26-29."""
    prefix = f"model.layers.{layer}."
    x = x + attention_block(x, W, prefix, c, positions, dense)
    h = rms_norm(x, W[prefix + "post_attention_layernorm.weight"], c["eps"])
    x = x + gated_mlp(h, W[prefix + "mlp.gate_proj.weight"],
                      W[prefix + "mlp.up_proj.weight"],
                      W[prefix + "mlp.down_proj.weight"])
    return x


def lm_head(x, W, c):
    """logits = norm(x) Wlm^T; tied models reuse the embedding table.
    crates/forward/src/core/composites/output_head.rs:32-57, 90-132;
    crates/models/qwen35-v2/src/loader.rs:219-223."""
    h = rms_norm(x, W["model.norm.weight"], c["eps"])
    head = W["model.embed_tokens.weight"] if c["tied"] or "lm_head.weight" not in W \
        else W["lm_head.weight"]
    return h @ head.T


# --------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------

def forward_logits(cfg: dict, W: dict, tokens, dense: bool = False, rows=None) -> torch.Tensor:
    """Logits [T, V] (float64) for one whole sequence at positions 0..T-1 (for the positions in `rows` only,
    if given; `dense` takes the masked-matrix form of the attention, for long sequences).
    crates/forward/README.md:18-39 gives the order of the parts."""
    c = _cfg(cfg)
    if not isinstance(W, LazyWeights):
        W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}
    positions = torch.arange(len(tokens))
    x = embedding(W["model.embed_tokens.weight"], tokens)
    for layer in range(c["L"]):
        x = decoder_block(x, W, layer, c, positions, dense)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    return lm_head(x, W, c)


def forward_logits_many(cfg: dict, W, sequences: dict, dense: bool = False) -> dict:
    """forward_logits for several whole sequences {name: tokens}, layer by layer over all of them, so that weights
    which are read when asked for (LazyWeights) are read once per layer and not once per sequence."""
    c = _cfg(cfg)
    emb = W["model.embed_tokens.weight"].to(F64)
    xs = {name: embedding(emb, toks) for name, toks in sequences.items()}
    del emb
    for layer in range(c["L"]):
        prefix = f"model.layers.{layer}."
        here = {k: W[k].to(F64) for k in W.keys() if k.startswith(prefix)}
        for name, toks in sequences.items():
            xs[name] = decoder_block(xs[name], here, layer, c, torch.arange(len(toks)), dense)
    tail = {k: W[k].to(F64) for k in ("model.norm.weight", "model.embed_tokens.weight", "lm_head.weight") if k in W}
    return {name: lm_head(x, tail, c) for name, x in xs.items()}


def argmax_lowest(row: torch.Tensor) -> int:
    """Strict '>' scan, so the lowest index wins a tie.
    crates/runtime/src/sampling.rs:486-496."""
    best, best_v = 0, -math.inf
    for i, v in enumerate(row.tolist()):
        if v > best_v:
            best, best_v = i, v
    return best


def greedy_generate(cfg: dict, W: dict, prompt, n_new: int) -> list[int]:
    """Prompt at [0, P), first generated token fed at position P."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward_logits(cfg, W, toks)
        t = argmax_lowest(logits[-1])
        out.append(t)
        toks.append(t)
    return out


# --------------------------------------------------------------------------
# sampling (host oracle)
# --------------------------------------------------------------------------

def softmax_temperature(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """softmax(logits / T) with max subtraction.
    crates/runtime/src/sampling.rs:610-640."""
    z = logits.to(F64) / temperature
    z = z - z.max()
    e = torch.exp(z)
    return e / e.sum()


def inverse_cdf_pick(probs: torch.Tensor, u: float) -> int:
    """u * sum, subtract probabilities in index order, first index where the
    remainder is <= 0. crates/runtime/src/sampling.rs:736-746."""
    r = u * float(probs.sum())
    for i, p in enumerate(probs.tolist()):
        r -= p
        if r <= 0.0:
            return i
    return len(probs) - 1


def apply_penalties(logits: torch.Tensor, history, repetition=1.0, presence=0.0,
                    frequency=0.0) -> torch.Tensor:
    """Repetition divides positive and multiplies negative logits of seen
    tokens; presence subtracts once; frequency subtracts count times.
    crates/runtime/src/sampling.rs:575-607."""
    out = logits.clone().to(F64)
    counts: dict[int, int] = {}
    for t in history:
        counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        if t >= len(out):
            continue
        if repetition != 1.0 and repetition > 0.0:
            out[t] = out[t] / repetition if out[t] > 0 else out[t] * repetition
        if presence != 0.0:
            out[t] -= presence
        if frequency != 0.0:
            out[t] -= frequency * c
    return out


def filtered_support(probs: torch.Tensor, top_k=None, top_p=None, min_p=None) -> list[int]:
    """Token ids that stay after top-k, then top-p (smallest sorted prefix whose
    mass reaches p), then min-p (drop below min_p * max).
    crates/runtime/src/sampling.rs:668-732."""
    order = sorted(range(len(probs)), key=lambda i: (-float(probs[i]), i))
    end = len(order)
    if top_k:
        end = min(end, int(top_k))
    if top_p is not None and 0.0 < top_p < 1.0:
        cum, pe = 0.0, 0
        for i in range(end):
            cum += float(probs[order[i]])
            pe = i + 1
            if cum >= top_p:
                break
        end = pe
    if min_p is not None and min_p > 0.0:
        thr = float(probs[order[0]]) * min_p
        drop = end
        for i in range(end):
            if float(probs[order[i]]) < thr:
                drop = i
                break
        end = max(drop, 1)
    return order[:end]
