"""What a step has to do, counted from the configuration: bytes it must read and flops it must perform.

These are the numerators of the roofline fractions: the algorithmic minimum (every weight once, the live cache
once, activations once in and once out), not what a kernel happens to move."""
from __future__ import annotations


def sizes(cfg) -> dict:
    qw = cfg.num_attention_heads * cfg.head_dim
    kvw = cfg.num_key_value_heads * cfg.head_dim
    return dict(H=cfg.hidden_size, I=cfg.intermediate_size, V=cfg.vocab_size, qw=qw, kvw=kvw,
                L=cfg.num_hidden_layers, window=cfg.sliding_window or 0)


def keys_seen(positions, window: int) -> int:
    """Sum over the query positions of the keys each sees: min(p + 1, W)."""
    return sum(min(p + 1, window) if window else p + 1 for p in positions)


def step_flops(cfg, layers: int, positions, n_out: int) -> float:
    """Flops of one step whose rows sit at `positions`: the linear maps of `layers` layers, attention over the
    visible keys (QK^T and PV, 2 flops per multiply-add), and the head on n_out rows."""
    s = sizes(cfg)
    n = len(positions)
    linear = 2.0 * n * layers * (s["H"] * (s["qw"] + 2 * s["kvw"]) + s["qw"] * s["H"] + 3 * s["H"] * s["I"])
    attention = 2.0 * 2.0 * keys_seen(positions, s["window"]) * s["qw"] * layers
    return linear + attention + 2.0 * n_out * s["V"] * s["H"]


def live_keys(context: int, window: int) -> int:
    return min(context, window) if window else context


def decode_step_bytes(weight_bytes: int, kv_bytes_per_token: int, contexts, window: int) -> int:
    """Every weight of the step once plus the cache of the live requests (what their windows still show)."""
    return weight_bytes + sum(live_keys(c, window) for c in contexts) * kv_bytes_per_token


def kernel_classes(cfg, rows: int, contexts, elem: int = 2, to_stream=None) -> dict:
    """For one layer call (and the head) of a step with `rows` rows whose sequences hold `contexts` tokens:
    class name -> dict(bytes, flops, matrix=(N, K) for the products).  `elem`: bytes of a weight or cache element.
    A step of decoded tokens has one row per context; a portion of a prompt has one context and `rows` rows that
    end at it."""
    s = sizes(cfg)
    H, I, V, qw, kvw, W = s["H"], s["I"], s["V"], s["qw"], s["kvw"], s["window"]

    def product(N, K, out_elem=4):
        return dict(bytes=N * K * elem + rows * K * elem + rows * N * out_elem, flops=2.0 * rows * N * K,
                    matrix=(N, K))

    if len(contexts) == rows:                                   # decoded tokens: each row reads its live cache
        seen = sum(live_keys(c, W) for c in contexts)
        attn_bytes = seen * 2 * kvw * elem + 2 * rows * qw * elem
    else:                                                       # a portion: keys are read once, queries see a triangle
        ctx = contexts[0]
        positions = range(ctx - rows, ctx)
        seen = keys_seen(positions, W)
        first_key = max(0, ctx - rows - W + 1) if W else 0
        attn_bytes = (ctx - first_key) * 2 * kvw * elem + 2 * rows * qw * elem
    # Over a portion in bfloat16 the output and down projections add to the residual stream themselves (read and
    # write it once, 8 bytes an element) and the norm after them reads the stream and writes the normalised rows;
    # else the projection writes float32, and the norm reads stream and projection and writes both.
    # (to_stream: whether they did; None: as the engine does for the benchmarked shapes at this row count)
    if to_stream is None:
        to_stream = rows > 512 and elem == 2
    norm_bytes = rows * H * ((4 + elem) if to_stream else (4 + 4 + 4 + elem))
    return {
        "qkv_proj": product(qw + 2 * kvw, H),
        "rotary_cache_write": dict(bytes=rows * (qw + 2 * kvw) * (4 + elem), flops=0.0),
        "attention": dict(bytes=attn_bytes, flops=4.0 * seen * qw),
        "o_proj": product(H, qw, out_elem=8 if to_stream else 4),
        "add_norm": dict(bytes=norm_bytes, flops=0.0),
        "gate_up_proj": dict(**product(2 * I, H, out_elem=elem), fused_activation=True),
        "gate_mul": dict(bytes=rows * I * (2 * 4 + elem), flops=0.0),
        "down_proj": product(H, I, out_elem=8 if to_stream else 4),
        "lm_head": dict(bytes=V * H * elem, flops=0.0, matrix=(V, H)),
    }
