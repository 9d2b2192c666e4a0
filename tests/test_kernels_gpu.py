"""The row-wise kernels and the sampler alone against plain torch float64 formulas, at sizes other than the
engine's (widths that are no power of two, odd row counts, every dtype combination the engine can meet)."""
import math

import pytest
import torch

import plain_mistral as pm

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"f": torch.float32, "b": torch.bfloat16}


def close(got, want, tol):
    err = float((got.double().cpu() - want.double().cpu()).abs().max())
    scale = float(want.double().abs().max()) or 1.0
    assert err / scale < tol, f"error {err / scale:.3e} of scale"


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("V,H,dt", [(11, 7, "f"), (300, 96, "b"), (1000, 4100, "b")])
def test_embedding(V, H, dt):
    from flambeau_b200.kernels import ops
    table = torch.randn(V, H, device=DEV).to(DT[dt])
    ids = torch.randint(0, V, (13,), dtype=torch.int32, device=DEV)
    x = torch.full((13, H), float("nan"), device=DEV)
    st = status()
    ops.embedding(table, ids, x, st)
    assert torch.equal(x, table[ids.long()].float()) and int(st.item()) == 0
    bad = ids.clone()
    bad[3] = V
    ops.embedding(table, bad, x, st)
    assert int(st.item()) == 1, "an id outside the table must be flagged"


@pytest.mark.parametrize("H", [8, 100, 96, 4096, 5120, 6000, 9216, 12288, 16384, 20000])
@pytest.mark.parametrize("dd,wd,od", ["fff", "fbb", "ffb", "bbb"])
def test_add_rms_norm(H, dd, wd, od):
    from flambeau_b200.kernels import ops
    n, eps = 5, 1e-5
    x = torch.randn(n, H, device=DEV)
    delta = (torch.randn(n, H, device=DEV) * 0.5).to(DT[dd])
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(DT[wd])
    out = torch.empty(n, H, device=DEV, dtype=DT[od])
    x0 = x.clone()
    ops.add_rms_norm(x, delta, w, eps, out)
    v = x0.double() + delta.double()
    close(x, v, 1e-6)                                             # the stream holds the sum
    close(out, pm.rms_norm(v, w.double(), eps), 2e-6 if od == "f" else 6e-3)
    # without a delta the stream is untouched
    x1 = x.clone()
    ops.add_rms_norm(x, None, w, eps, out)
    assert torch.equal(x, x1)
    close(out, pm.rms_norm(x1.double(), w.double(), eps), 2e-6 if od == "f" else 6e-3)


def test_add_rms_norm_rows_and_slabs():
    from flambeau_b200.kernels import ops
    n, H, eps, P = 9, 200, 1e-6, 7
    x = torch.randn(n, H, device=DEV)
    slabs = torch.randn(P, n, H, device=DEV)
    w = torch.randn(H, device=DEV)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, H, device=DEV)
    x0 = x.clone()
    ops.add_rms_norm(x, slabs[0], w, eps, out, rows=rows, n_partials=5, partial_stride=slabs.stride(0))
    assert torch.equal(x, x0), "with a row list the stream is read only"
    v = (x0.double() + slabs[:5].double().sum(0))[rows.long()]
    close(out, pm.rms_norm(v, w.double(), eps), 3e-6)
    out_all = torch.empty(n, H, device=DEV)
    ops.add_rms_norm(x, slabs[0], w, eps, out_all, n_partials=P, partial_stride=slabs.stride(0))
    close(x, x0.double() + slabs.double().sum(0), 2e-6)


@pytest.mark.parametrize("n,H,P", [(1, 1024, 1), (8, 4096, 16), (3, 2048, 5), (64, 4096, 8), (8, 5120, 20),
                                   (300, 4096, 3), (200, 5120, 2), (130, 2048, 5), (150, 8192, 2), (129, 16384, 2)])
@pytest.mark.parametrize("od", ["f", "b"])
def test_add_rms_norm_few_wide_rows(n, H, P, od):
    """The widths of real models with the row counts of decoding, and as many split-K slabs as the products leave;
    and the same over the hundreds of rows of a portion whose product left shares (a launch shape of its own)."""
    from flambeau_b200.kernels import ops
    eps = 1e-5
    g = torch.Generator(device=DEV).manual_seed(n * H + P)
    x = torch.randn(n, H, device=DEV, generator=g)
    slabs = torch.randn(P, n, H, device=DEV, generator=g) * 0.3
    w = (1 + 0.1 * torch.randn(H, device=DEV, generator=g)).to(DT[od])
    out = torch.empty(n, H, device=DEV, dtype=DT[od])
    x0 = x.clone()
    ops.add_rms_norm(x, slabs[0], w, eps, out, n_partials=P, partial_stride=slabs.stride(0))
    v = x0.double() + slabs.double().sum(0)
    close(x, v, 2e-6)
    close(out, pm.rms_norm(v, w.double(), eps), 3e-6 if od == "f" else 6e-3)
    rows = torch.tensor([n - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, device=DEV, dtype=DT[od])
    x1 = x.clone()
    ops.add_rms_norm(x, None, w, eps, out2, rows=rows)
    assert torch.equal(x, x1)
    close(out2, pm.rms_norm(x1.double()[rows.long()], w.double(), eps), 3e-6 if od == "f" else 6e-3)


@pytest.mark.parametrize("n,H", [(257, 128), (300, 1024), (513, 4096), (258, 5120), (259, 8192), (260, 4100), (261, 9216)])
@pytest.mark.parametrize("dd,od", [("f", "f"), ("f", "b"), ("b", "b")])
def test_add_rms_norm_many_rows(n, H, dd, od):
    """A prompt's portion: hundreds of rows with one delta each, at widths that take each of the kernel's forms
    (several rows per block, two vectors per thread, and the widths that neither takes), with an odd row count."""
    from flambeau_b200.kernels import ops
    eps = 1e-5
    g = torch.Generator(device=DEV).manual_seed(n + H)
    x = torch.randn(n, H, device=DEV, generator=g)
    x[n - 1] *= 7.0                                              # the last row stands out: a block that took its
    x[n - 2] *= 0.01                                             # neighbour's sum of squares would show
    delta = (torch.randn(n, H, device=DEV, generator=g) * 0.5).to(DT[dd])
    w = (1 + 0.1 * torch.randn(H, device=DEV, generator=g)).to(DT[od])
    out = torch.empty(n, H, device=DEV, dtype=DT[od])
    x0 = x.clone()
    ops.add_rms_norm(x, delta, w, eps, out)
    v = x0.double() + delta.double()
    close(x, v, 1e-6)
    close(out, pm.rms_norm(v, w.double(), eps), 3e-6 if od == "f" else 6e-3)
    # nothing to add (the stream holds the sum already): the same rows, normalised, the stream untouched
    x1 = x.clone()
    out.fill_(float("nan"))
    ops.add_rms_norm(x, None, w, eps, out)
    assert torch.equal(x, x1)
    close(out, pm.rms_norm(x1.double(), w.double(), eps), 3e-6 if od == "f" else 6e-3)


@pytest.mark.parametrize("half,theta", [(8, 1e4), (12, 1e6), (64, 1e4)])
def test_rope_table_is_right_at_far_positions(half, theta):
    from flambeau_b200.kernels import ops
    pos = torch.tensor([0, 1, 17, 4095, 8191, 131071, 1000003], dtype=torch.int32, device=DEV)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / (2 * half))
    cos = torch.empty(len(pos), half, device=DEV)
    sin = torch.empty(len(pos), half, device=DEV)
    ops.rope_table(pos, inv.to(DEV), cos, sin)
    ang = pos.double().cpu()[:, None] * inv[None, :]
    assert float((cos.cpu().double() - torch.cos(ang)).abs().max()) < 1e-6
    assert float((sin.cpu().double() - torch.sin(ang)).abs().max()) < 1e-6


@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (8, 1, 24, 24), (3, 3, 40, 16), (32, 8, 128, 128)])
@pytest.mark.parametrize("dt_in,dt_out,slabs", [("f", "f", 1), ("f", "b", 1), ("f", "b", 6), ("b", "b", 1)])
def test_rope_and_cache_write(nh, nkv, hd, rot, dt_in, dt_out, slabs):
    from flambeau_b200.kernels import ops
    n, ps, n_pages, theta = 11, 8, 9, 1e4
    half = rot // 2
    g = torch.Generator(device=DEV).manual_seed(nh + hd)
    width = (nh + 2 * nkv) * hd
    parts = (torch.randn(slabs, n, width, device=DEV, generator=g)).to(DT[dt_in])
    whole = parts.double().sum(0)
    positions = torch.tensor([3, 4, 5, 6, 7, 8, 40, 0, 1, 2, 63], dtype=torch.int32, device=DEV)
    row_seq = torch.tensor([0] * 6 + [1] + [2] * 3 + [1], dtype=torch.int32, device=DEV)
    table = torch.full((3, 8), -1, dtype=torch.int32, device=DEV)
    table[0, 0], table[0, 1] = 5, 2
    table[1, 5], table[1, 7] = 0, 7
    table[2, 0] = 3
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / rot)
    cos = torch.empty(n, half, device=DEV)
    sin = torch.empty(n, half, device=DEV)
    ops.rope_table(positions, inv.to(DEV), cos, sin)
    kp = torch.zeros(n_pages, nkv, ps, hd, device=DEV, dtype=DT[dt_out])
    vp = torch.zeros_like(kp)
    q_out = torch.empty(n, nh * hd, device=DEV, dtype=DT[dt_out])
    st = status()
    qkv = parts[0]
    ops.rope_kv_write(qkv[:, :nh * hd], q_out, qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:], cos, sin,
                      half, positions, row_seq, table, kp, vp, ps, nh, nkv, hd, True, st,
                      n_partials=slabs, partial_stride=parts.stride(0))
    assert int(st.item()) == 0
    q = whole[:, :nh * hd].reshape(n, nh, hd)
    k = whole[:, nh * hd:(nh + nkv) * hd].reshape(n, nkv, hd)
    v = whole[:, (nh + nkv) * hd:].reshape(n, nkv, hd)
    tol = 2e-6 if dt_out == "f" else 5e-3
    close(q_out.reshape(n, nh, hd), pm.rope_split_half(q.cpu(), positions.cpu(), theta, rot), tol)
    k_rot = pm.rope_split_half(k.cpu(), positions.cpu(), theta, rot)
    for r in range(n):
        p, s = int(positions[r]), int(row_seq[r])
        page = int(table[s, p // ps])
        close(kp[page, :, p % ps], k_rot[r], tol)
        close(vp[page, :, p % ps], v[r].cpu(), tol)
    written = sum(1 for _ in range(n))
    assert int((kp.float().abs().sum(dim=(1, 3)) > 0).sum()) == written, "only the rows of the step are written"


@pytest.mark.parametrize("nh,nkv,hd,rot", [(3, 3, 40, 16), (32, 8, 128, 128)])
@pytest.mark.parametrize("dt_out", ["f", "b"])
def test_rope_and_cache_write_of_a_long_portion(nh, nkv, hd, rot, dt_out):
    """Over a thousand tokens in one call (an odd count, three sequences, pages in a shuffled order): the form of
    the kernel that takes several tokens per thread."""
    from flambeau_b200.kernels import ops
    ps, theta = 8, 1e4
    lens = [700, 3, 326]
    starts = [5, 0, 1000]
    n = sum(lens)
    half = rot // 2
    g = torch.Generator(device=DEV).manual_seed(nh * hd)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(n, width, device=DEV, generator=g)
    positions = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lens)]).int().to(DEV)
    row_seq = torch.cat([torch.full((l,), i) for i, l in enumerate(lens)]).int().to(DEV)
    per_seq = max(-(-(s + l) // ps) for s, l in zip(starts, lens))
    n_pages = 3 * per_seq
    table = torch.randperm(n_pages, device=DEV, generator=g).int().view(3, per_seq)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / rot)
    cos = torch.empty(n, half, device=DEV)
    sin = torch.empty(n, half, device=DEV)
    ops.rope_table(positions, inv.to(DEV), cos, sin)
    kp = torch.zeros(n_pages, nkv, ps, hd, device=DEV, dtype=DT[dt_out])
    vp = torch.zeros_like(kp)
    q_out = torch.empty(n, nh * hd, device=DEV, dtype=DT[dt_out])
    st = status()
    ops.rope_kv_write(qkv[:, :nh * hd], q_out, qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:], cos, sin,
                      half, positions, row_seq, table, kp, vp, ps, nh, nkv, hd, True, st)
    assert int(st.item()) == 0
    q = qkv[:, :nh * hd].reshape(n, nh, hd).double().cpu()
    k = qkv[:, nh * hd:(nh + nkv) * hd].reshape(n, nkv, hd).double().cpu()
    v = qkv[:, (nh + nkv) * hd:].reshape(n, nkv, hd).double().cpu()
    tol = 2e-6 if dt_out == "f" else 5e-3
    close(q_out.reshape(n, nh, hd), pm.rope_split_half(q, positions.cpu(), theta, rot), tol)
    page = table.cpu().long()[row_seq.cpu().long(), (positions.cpu() // ps).long()]
    slot = (positions.cpu() % ps).long()
    close(kp.cpu()[page, :, slot], pm.rope_split_half(k, positions.cpu(), theta, rot), tol)
    close(vp.cpu()[page, :, slot], v, tol)
    assert int((kp.float().abs().sum(dim=(1, 3)) > 0).sum()) == n, "only the rows of the step are written"


def test_cache_write_flags_a_missing_page():
    from flambeau_b200.kernels import ops
    qkv = torch.randn(2, 4 * 16, device=DEV)
    q_out = torch.empty(2, 2 * 16, device=DEV)
    kp = torch.zeros(2, 1, 8, 16, device=DEV)
    table = torch.full((1, 4), -1, dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    st = status()
    ops.rope_kv_write(qkv[:, :32], q_out, qkv[:, 32:48], qkv[:, 48:], None, None, 0, pos, torch.zeros_like(pos), table,
                      kp, torch.zeros_like(kp), 8, 2, 1, 16, True, st)
    assert int(st.item()) == 2


def gate_times(activation, g, u):
    """The gate activations of the kernels, in float64."""
    if activation == "silu":
        return g / (1 + torch.exp(-g)) * u
    return 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))) * u


@pytest.mark.parametrize("n,I", [(1, 7), (5, 160), (3, 14336), (2, 1002)])
@pytest.mark.parametrize("di,do,slabs", [("f", "f", 1), ("b", "b", 1), ("f", "b", 5), ("f", "b", 9)])
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_gate_mul(n, I, di, do, slabs, activation):
    from flambeau_b200.kernels import ops
    parts = torch.randn(slabs, n, 2 * I, device=DEV).to(DT[di])
    out = torch.empty(n, I, device=DEV, dtype=DT[do])
    ops.gate_mul(parts[0], out, n_partials=slabs, partial_stride=parts.stride(0), activation=activation)
    gu = parts.double().sum(0)
    g, u = gu[:, 0::2], gu[:, 1::2]                         # gate and up alternate along a row
    close(out, gate_times(activation, g, u), 3e-6 if do == "f" else 6e-3)


def test_an_unknown_activation_is_refused():
    from flambeau_b200.kernels import ops
    from flambeau_b200.kernels.library import KernelError
    gu = torch.randn(2, 8, device=DEV)
    with pytest.raises(KernelError, match="not implemented"):
        ops.gate_mul(gu, torch.empty(2, 4, device=DEV), activation="relu")


@pytest.mark.parametrize("n,H,od", [(3, 96, "f"), (5, 4096, "b"), (300, 1024, "b"), (2, 20000, "f")])
def test_add_rms_norm_with_a_weight_offset(n, H, od):
    """The "1 + w" form of the norm: the stored weight plus an offset, in each of the kernel's forms."""
    from flambeau_b200.kernels import ops
    eps = 1e-6
    x = torch.randn(n, H, device=DEV)
    delta = torch.randn(n, H, device=DEV) * 0.5
    w = (0.1 * torch.randn(H, device=DEV)).to(DT[od])
    out = torch.empty(n, H, device=DEV, dtype=DT[od])
    x0 = x.clone()
    ops.add_rms_norm(x, delta, w, eps, out, weight_offset=1.0)
    v = x0.double() + delta.double()
    close(out, pm.rms_norm(v, 1.0 + w.double(), eps), 3e-6 if od == "f" else 6e-3)


def test_cache_write_through_a_table_that_starts_at_a_later_page():
    """A table row holds live pages only: column 0 stands for the logical page given in table_base."""
    from flambeau_b200.kernels import ops
    ps, nkv, hd, nh = 8, 2, 16, 2
    positions = torch.tensor([100, 101, 7, 103], dtype=torch.int32, device=DEV)
    row_seq = torch.tensor([0, 0, 1, 0], dtype=torch.int32, device=DEV)
    table = torch.tensor([[5, 3, -1], [9, -1, -1]], dtype=torch.int32, device=DEV)
    base = torch.tensor([11, 0], dtype=torch.int32, device=DEV)          # sequence 0: columns are pages 11, 12, 13
    qkv = torch.randn(4, (nh + 2 * nkv) * hd, device=DEV)
    kp = torch.zeros(12, nkv, ps, hd, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.empty(4, nh * hd, device=DEV)
    st = status()
    ops.rope_kv_write(qkv[:, :nh * hd], q_out, qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:], None, None,
                      0, positions, row_seq, table, kp, vp, ps, nh, nkv, hd, True, st, table_base=base)
    assert int(st.item()) == 0
    k = qkv[:, nh * hd:(nh + nkv) * hd].reshape(4, nkv, hd)
    for r, (page, slot) in enumerate([(3, 4), (3, 5), (9, 7), (3, 7)]):
        assert torch.equal(kp[page, :, slot], k[r])
    # a position below the row's first page has no column: flagged, nothing written
    positions[0] = 80
    ops.rope_kv_write(qkv[:, :nh * hd], q_out, qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:], None, None,
                      0, positions, row_seq, table, kp, vp, ps, nh, nkv, hd, True, st, table_base=base)
    assert int(st.item()) == 2


# ---- sampler -------------------------------------------------------------------------------------------------

def test_argmax_takes_the_lowest_index_of_a_tie():
    from flambeau_b200.kernels import ops
    V = 70001
    logits = torch.randn(4, V, device=DEV)
    logits[0, 123] = logits[0, 60000] = 50.0
    logits[1, :] = 1.0
    logits[2, V - 1] = 99.0
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.sample(logits, out)
    want = [pm.argmax_lowest(r) for r in logits.cpu()]
    assert out.tolist() == want and want[0] == 123 and want[1] == 0 and want[2] == V - 1


@pytest.mark.parametrize("V", [320, 32000, 131072 + 5])
def test_temperature_draw_is_the_inverse_cdf(V):
    from flambeau_b200.kernels import ops
    n = 16
    g = torch.Generator(device=DEV).manual_seed(V)
    logits = torch.randn(n, V, device=DEV, generator=g) * 3
    temp = torch.tensor([0.0, 0.5, 0.8, 1.0, 1.5, 0.3, 2.0, 1.0] * 2, device=DEV)
    u = torch.tensor([0.0, 0.999, 0.5, 0.25, 0.75, 0.1, 0.9, 0.33] * 2, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, temperature=temp, uniform=u)
    for r in range(n):
        row = logits[r].cpu()
        if float(temp[r]) <= 0:
            assert int(out[r]) == pm.argmax_lowest(row)
            continue
        p = pm.softmax_temperature(row, float(temp[r]))
        cdf = torch.cumsum(p, 0)
        tok = int(out[r])
        lo = float(cdf[tok - 1]) if tok else 0.0
        # float32 sums on the device: the drawn token's CDF interval must hold u within a small slack
        assert lo - 1e-4 <= float(u[r]) <= float(cdf[tok]) + 1e-4, f"row {r}: token {tok} does not hold u"


def test_filters_keep_the_reference_support():
    from flambeau_b200.kernels import ops
    V, n = 5000, 6
    g = torch.Generator(device=DEV).manual_seed(1)
    logits = torch.randn(n, V, device=DEV, generator=g) * 2.5
    cfgs = [dict(top_k=5), dict(top_p=0.6), dict(min_p=0.2), dict(top_k=50, top_p=0.9), dict(top_k=3, min_p=0.5),
            dict(top_p=0.3, min_p=0.05)]
    T = 0.9
    for trial in range(40):
        u = torch.rand(n, device=DEV, generator=g)
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        ops.sample(logits, out, temperature=torch.full((n,), T, device=DEV), uniform=u,
                   top_k=torch.tensor([c.get("top_k", 0) for c in cfgs], dtype=torch.int32, device=DEV),
                   top_p=torch.tensor([c.get("top_p", 0.0) for c in cfgs], device=DEV),
                   min_p=torch.tensor([c.get("min_p", 0.0) for c in cfgs], device=DEV))
        for r, c in enumerate(cfgs):
            probs = pm.softmax_temperature(logits[r].cpu(), T)
            support = set(pm.filtered_support(probs, **c))
            assert int(out[r]) in support, f"{c}: token {int(out[r])} is outside the kept set of {len(support)}"
    # a draw with u close to 0 returns the lowest kept index, close to 1 the highest
    probs = pm.softmax_temperature(logits[0].cpu(), T)
    support = sorted(pm.filtered_support(probs, top_k=5))
    for uval, want in ((0.0, support[0]), (0.99999, support[-1])):
        out = torch.empty(1, dtype=torch.int32, device=DEV)
        ops.sample(logits[:1], out, temperature=torch.tensor([T], device=DEV), uniform=torch.tensor([uval], device=DEV),
                   top_k=torch.tensor([5], dtype=torch.int32, device=DEV), top_p=torch.zeros(1, device=DEV),
                   min_p=torch.zeros(1, device=DEV))
        assert int(out[0]) == want


def test_penalties_and_bias():
    from flambeau_b200.kernels import ops
    V = 100
    logits = torch.randn(2, V, device=DEV)
    before = logits.clone().cpu()
    history = [[3, 3, 7, 99], [5]]
    rows, toks, cnts = [], [], []
    for r, h in enumerate(history):
        for t in sorted(set(h)):
            rows.append(r); toks.append(t); cnts.append(h.count(t))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    ops.apply_penalties(logits, i32(rows), i32(toks), i32(cnts), f32([1.3, 1.0]), f32([0.4, 0.0]), f32([0.1, 0.7]))
    want0 = pm.apply_penalties(before[0], history[0], repetition=1.3, presence=0.4, frequency=0.1)
    want1 = pm.apply_penalties(before[1], history[1], repetition=1.0, presence=0.0, frequency=0.7)
    close(logits[0], want0, 1e-6)
    close(logits[1], want1, 1e-6)
    ops.apply_logit_bias(logits, i32([0, 1]), i32([10, 20]), f32([5.0, -2.0]))
    assert math.isclose(float(logits[0, 10]), float(want0[10]) + 5.0, rel_tol=1e-6)
    assert math.isclose(float(logits[1, 20]), float(want1[20]) - 2.0, rel_tol=1e-6)
