"""The attention kernels alone against a plain softmax over gathered keys, at sizes other than the engine's:
float32 CUDA-core kernel and bfloat16 tensor-core kernel; grouped heads 1:1, 2:1, 4:1, 8:1; head sizes from 16
to 256; windows; pages in random order, pages of the prefix taken back; portions beside decoded tokens in one
call; and single keys that stand out at the edge of a page, of a window and of a chunk."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


class Scene:
    """A set of sequences with keys/values scattered over a paged pool, plus this step's queries."""

    def __init__(self, seqs, nh, nkv, hd, window, dtype, page_size=16, seed=0, spread=1.0, extra_pages=7, ramp=0.0,
                 compact=False):
        # seqs: list of (cached tokens before the step, new tokens in the step)
        # compact: a table row holds the live pages only and starts at the sequence's first live page (what the
        # engine's cache manager hands out); else rows start at page 0 and pages given back are -1 entries
        g = torch.Generator().manual_seed(seed)
        rnd = random.Random(seed)
        self.nh, self.nkv, self.hd, self.window, self.dtype, self.ps = nh, nkv, hd, window, dtype, page_size
        self.slopes = None            # per query head: slope * (key position - query position) added to the scores
        self.seqs = seqs
        total_pages = sum(-(-(a + b) // page_size) for a, b in seqs) + extra_pages
        ids = list(range(total_pages))
        rnd.shuffle(ids)
        def first_page(cached):                     # the first page the cache manager still holds
            return (max(0, cached - window + 1) // page_size) if (window and compact) else 0
        max_pages = max(-(-(a + b) // page_size) - first_page(a) for a, b in seqs) + 2
        self.k_pool = torch.full((total_pages, nkv, page_size, hd), float("nan"))   # unwritten slots are poison
        self.v_pool = torch.full((total_pages, nkv, page_size, hd), float("nan"))
        self.table = torch.full((len(seqs), max_pages), -1, dtype=torch.int32)
        self.table_base = torch.zeros(len(seqs), dtype=torch.int32) if compact else None
        self.k, self.v, self.q = [], [], []
        rows = []
        for s, (cached, new) in enumerate(seqs):
            T = cached + new
            k = torch.randn(T, nkv, hd, generator=g) * spread
            if ramp:                                                    # later keys score higher and higher
                k = k * (1.0 + ramp * torch.arange(T, dtype=torch.float32)).view(T, 1, 1)
            v = torch.randn(T, nkv, hd, generator=g)
            q = torch.randn(new, nh, hd, generator=g) * spread
            k, v, q = (t.to(dtype).float() for t in (k, v, q))          # values exactly representable in dtype
            self.k.append(k); self.v.append(v); self.q.append(q)
            first_live = max(0, cached - window + 1) if window else 0   # what the cache manager keeps
            base = first_live // page_size if compact else 0
            if compact:
                self.table_base[s] = base
            for j in range(-(-T // page_size)):
                if (j + 1) * page_size <= first_live:
                    continue                                            # page given back: table stays -1
                pid = ids.pop()
                self.table[s, j - base] = pid
                lo, hi = j * page_size, min(T, (j + 1) * page_size)
                self.k_pool[pid, :, :hi - lo] = k[lo:hi].transpose(0, 1)
                self.v_pool[pid, :, :hi - lo] = v[lo:hi].transpose(0, 1)
            rows += [(s, cached + i) for i in range(new)]
        self.rows = rows
        self.positions = torch.tensor([p for _, p in rows], dtype=torch.int32)
        self.row_seq = torch.tensor([s for s, _ in rows], dtype=torch.int32)
        self.q_flat = torch.cat(self.q).reshape(len(rows), nh * hd)
        starts, acc = [], 0
        for _, new in seqs:
            starts.append(acc)
            acc += new
        self.seq_q_start = torch.tensor(starts, dtype=torch.int32)
        self.seq_q_len = torch.tensor([n for _, n in seqs], dtype=torch.int32)
        self.seq_pos_start = torch.tensor([c for c, _ in seqs], dtype=torch.int32)

    def reference(self, scale):
        out = torch.zeros(len(self.rows), self.nh, self.hd, dtype=torch.float64)
        G = self.nh // self.nkv
        i = 0
        for s, (cached, new) in enumerate(self.seqs):
            k, v, q = self.k[s].double(), self.v[s].double(), self.q[s].double()
            for j in range(new):
                p = cached + j
                t0 = max(0, p - self.window + 1) if self.window else 0
                for h in range(self.nh):
                    sc = scale * (k[t0:p + 1, h // G] @ q[j, h])
                    if self.slopes is not None:
                        sc = sc + float(self.slopes[h]) * (torch.arange(t0, p + 1, dtype=torch.float64) - p)
                    w = torch.softmax(sc, dim=0)
                    out[i, h] = w @ v[t0:p + 1, h // G]
                i += 1
        return out.reshape(len(self.rows), self.nh * self.hd)

    def page_of(self, s, position):
        """Physical page of a position of sequence s (-1: given back)."""
        base = int(self.table_base[s]) if self.table_base is not None else 0
        return int(self.table[s, position // self.ps - base])

    def run(self, kernel, scale, prefetch=None):
        from flambeau_b200.kernels import ops
        dev = "cuda"
        q = self.q_flat.to(dev, self.dtype)
        out = torch.full_like(q, float("nan"))
        kp, vp = self.k_pool.to(dev, self.dtype), self.v_pool.to(dev, self.dtype)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        table = self.table.to(dev)
        base = self.table_base.to(dev) if self.table_base is not None else None
        slopes = self.slopes.to(dev, torch.float32) if self.slopes is not None else None
        if kernel == "simt":
            ops.paged_attention_simt(q, out, kp, vp, table, self.positions.to(dev), self.row_seq.to(dev),
                                     self.nh, self.nkv, self.hd, self.window, scale, status, table_base=base,
                                     score_slopes=slopes)
        else:
            G = self.nh // self.nkv
            short = [n * G <= 16 for _, n in self.seqs]
            assert ops.mma_attention_supported(q, self.nh, self.nkv, self.hd)
            multi = [s for s, (_, n) in enumerate(self.seqs) if n > 1]      # as the engine's descriptor lists them
            multi_d = torch.tensor(multi + [0], dtype=torch.int32, device=dev)
            ops.paged_attention_mma(q, out, kp, vp, table, self.seq_q_start.to(dev), self.seq_q_len.to(dev),
                                    self.seq_pos_start.to(dev), len(self.seqs), max(n for _, n in self.seqs),
                                    max(c + n for c, n in self.seqs), any(short), not all(short), self.nh, self.nkv,
                                    self.hd, self.window, scale, status, table_base=base, prefetch=prefetch,
                                    multi_seqs=multi_d, n_multi=len(multi), score_slopes=slopes)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, "the kernel flagged a fault (missing page or timed-out wait)"
        return out.float().cpu()


def check(scene, kernel, tol=None):
    scale = 1.0 / math.sqrt(scene.hd)
    got, want = scene.run(kernel, scale), scene.reference(scale)
    assert torch.isfinite(got).all(), "poison from an unwritten or released slot reached the output"
    tol = tol if tol is not None else (2e-5 if scene.dtype == torch.float32 else 1.2e-2)
    err = float((got.double() - want).abs().max() / want.abs().max())
    assert err < tol, f"{kernel}: error {err:.3e}"


KERNELS = [("simt", torch.float32), ("simt", torch.bfloat16), ("mma", torch.bfloat16)]
GEOMETRY = [(4, 4, 16), (4, 2, 24), (8, 2, 64), (8, 1, 80), (32, 8, 128), (6, 3, 40), (2, 1, 256), (16, 2, 32),
            (32, 1, 64)]       # the last: 32 query heads on one key/value head, where even a single token is "long"


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("nh,nkv,hd", GEOMETRY)
@pytest.mark.parametrize("window", [0, 24])
def test_portions_beside_decoded_tokens(kernel, dtype, nh, nkv, hd, window):
    seqs = [(0, 37), (50, 1), (3, 2), (129, 1), (17, 70), (0, 1), (64, 3), (200, 1)]
    check(Scene(seqs, nh, nkv, hd, window, dtype, seed=nh * 100 + hd + window), kernel)


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 24), (8, 2, 64), (32, 8, 128), (32, 1, 64)])
@pytest.mark.parametrize("window", [0, 40])
def test_a_penalty_on_distance_per_head(kernel, dtype, nh, nkv, hd, window):
    """slope_h * (key position - query position) added to the scores: slopes that differ from head to head and are
    steep enough to change which keys count (the nearest few for the steepest head, all of them for slope 0);
    decoded tokens at several depths beside portions, so the split-key and the portion arrangements both run."""
    sc = Scene([(300, 1), (0, 37), (130, 1), (75, 20), (11, 1)], nh, nkv, hd, window, dtype, seed=nh + hd + window,
               spread=0.5)
    sc.slopes = torch.tensor([0.0 if h == 0 else 2.0 ** (-8.0 * h / nh) for h in range(nh)], dtype=torch.float64)
    check(sc, kernel)
    plain = Scene([(300, 1), (0, 37), (130, 1), (75, 20), (11, 1)], nh, nkv, hd, window, dtype, seed=nh + hd + window,
                  spread=0.5)
    scale = 1.0 / math.sqrt(hd)
    moved = (sc.reference(scale) - plain.reference(scale)).abs().max() / plain.reference(scale).abs().max()
    assert moved > 0.05, "the slopes of this test do not move the result: it could not fail"


def test_slopes_must_be_one_float_per_head():
    from flambeau_b200.kernels import ops
    from flambeau_b200.kernels.library import KernelError
    sc = Scene([(20, 1)], 4, 2, 32, 0, torch.bfloat16)
    sc.slopes = torch.zeros(3, dtype=torch.float64)
    with pytest.raises(KernelError, match="one per query head"):
        sc.run("mma", 0.1)


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("page_size", [8, 16, 64])
def test_long_context_many_chunks(kernel, dtype, page_size):
    # long enough that the split-key arrangement uses many chunks, and that a portion spans many key tiles
    seqs = [(3000, 1), (777, 1), (1500, 130), (4095, 2)]
    check(Scene(seqs, 8, 2, 64, 0, dtype, page_size=page_size, seed=page_size), kernel)
    check(Scene(seqs, 8, 2, 64, 1000, dtype, page_size=page_size, seed=page_size + 1), kernel)


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("where", ["page_edge_low", "page_edge_high", "window_first", "just_outside_window",
                                   "first_key", "self", "chunk_edge"])
def test_one_key_stands_out(kernel, dtype, where):
    """Scale one key so that its score dominates: the output must be that key's value (or must not be, when the
    key lies just outside the window).  A kernel that drops or adds a key at an edge fails by a wide margin."""
    window, cached, nh, nkv, hd = 100, 700, 4, 2, 32
    p = cached                       # the single query's position
    target = {"page_edge_low": 640, "page_edge_high": 655, "window_first": p - window + 1,
              "just_outside_window": p - window, "first_key": 0, "self": p, "chunk_edge": 639}[where]
    if where == "first_key":
        window = 0
    sc = Scene([(cached, 1), (40, 1)], nh, nkv, hd, window, dtype, seed=5, spread=0.3)
    for h in range(nkv):
        qh = sc.q[0][0, h * (nh // nkv)]
        sc.k[0][target, h] = (qh / qh.norm() * 40.0).to(dtype).float()      # score ~ 40*|q|/sqrt(hd) >> others
    # rewrite the pool with the planted key
    slot = target % 16
    pid = sc.page_of(0, target)
    if pid >= 0:
        sc.k_pool[pid, :, slot] = sc.k[0][target]
    scale = 1.0 / math.sqrt(hd)
    got = sc.run(kernel, scale).reshape(-1, nh, hd)
    want = sc.reference(scale).reshape(-1, nh, hd)
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    assert float((got.double() - want).abs().max() / want.abs().max()) < tol
    planted = sc.v[0][target]                                               # [nkv, hd]
    head0 = got[0, 0]
    closeness = float((head0 - planted[0]).abs().max())
    if where == "just_outside_window":
        assert closeness > 0.3, "a key outside the window was attended to"
    else:
        # heads whose query the key was built from see (almost) only that key ("self": the query's own key,
        # written by this step, at the last slot the query may see)
        assert closeness < 0.05, "the key that dominates was lost"


@pytest.mark.parametrize("nh,nkv,hd,page_size", [(8, 2, 64, 16), (6, 3, 40, 8), (4, 1, 128, 32)])
@pytest.mark.parametrize("window", [0, 300])
def test_many_decoded_sequences_of_unequal_length(nh, nkv, hd, page_size, window):
    """Forty decoded tokens with contexts from one key to a few thousand: the split-key kernel cuts the line of all
    their key tiles into equal stretches, so a CTA's stretch ends inside one sequence, runs over several short ones
    and starts inside another; every result must still be the plain softmax over that sequence's own keys."""
    rnd = random.Random(hd + window)
    seqs = [(rnd.choice([0, 1, 15, 63, 64, 65, 127, 128, 500, 1000, 2100]) + rnd.randrange(3), rnd.choice([1, 1, 1, 2]))
            for _ in range(40)]
    check(Scene(seqs, nh, nkv, hd, window, torch.bfloat16, page_size=page_size, seed=hd + window), "mma")


def test_steps_of_different_shapes_alternate():
    """The split-key kernel keeps counters and partial results in one scratch buffer between launches; steps of
    other head sizes and batch sizes in between must leave it usable (each scene is checked twice)."""
    scenes = [Scene([(900, 1), (70, 1), (2500, 2)], 8, 2, 128, 0, torch.bfloat16, seed=1),
              Scene([(300, 1)] * 9, 4, 4, 32, 0, torch.bfloat16, seed=2),
              Scene([(1200, 1), (5, 1)], 16, 2, 64, 500, torch.bfloat16, page_size=8, seed=3)]
    for _ in range(2):
        for sc in scenes:
            check(sc, "mma")


@pytest.fixture(params=[True, False], ids=["tcgen05", "mma_sync"])
def prompt_kernel(request):
    """Portions of prompts on the tcgen05 kernel (where it takes the geometry) and on the mma.sync kernel."""
    from flambeau_b200.kernels import ops
    ops.set_attention_tc(request.param)
    yield request.param
    ops.set_attention_tc(True)


@pytest.mark.parametrize("nh,nkv,hd,page_size", [(8, 2, 128, 16), (8, 2, 64, 8), (4, 4, 128, 64), (6, 3, 64, 32),
                                                  (16, 1, 128, 16)])
@pytest.mark.parametrize("window", [0, 300])
def test_whole_prompts_and_late_portions(prompt_kernel, nh, nkv, hd, page_size, window):
    """Prompts over several 128-key tiles, from position 0 and after a cached prefix, beside a decoded token;
    token counts that fill no tile of rows; grouped heads 1, 2, 4 and 16."""
    seqs = [(0, 700), (900, 131), (415, 1), (250, 7)]
    check(Scene(seqs, nh, nkv, hd, window, torch.bfloat16, page_size=page_size, seed=hd + window + nh), "mma")


def test_scores_that_grow_along_the_keys(prompt_kernel):
    """Keys whose scores rise with the position: the running maximum of a row grows from tile to tile by more than
    the step at which the tcgen05 kernel moves its reference point, so the accumulated output is rescaled there."""
    sc = Scene([(0, 900), (100, 400)], 8, 2, 128, 0, torch.bfloat16, seed=11, spread=1.0, ramp=0.03)
    check(sc, "mma")


def test_one_far_key_among_a_long_prompt(prompt_kernel):
    """One key of a 1,000-token prompt is scaled so that the last tokens' queries of its group see (almost) only
    it: a tile that is dropped, fetched from the wrong page or multiplied with the wrong value rows shows."""
    nh, nkv, hd = 8, 2, 128
    for target in (0, 127, 128, 517, 895):
        sc = Scene([(0, 1000)], nh, nkv, hd, 0, torch.bfloat16, seed=target, spread=0.3)
        for h in range(nkv):
            qh = sc.q[0][-1, h * (nh // nkv)]
            sc.k[0][target, h] = (qh / qh.norm() * 100.0).to(torch.bfloat16).float()
        pid = sc.page_of(0, target)
        sc.k_pool[pid, :, target % 16] = sc.k[0][target]
        scale = 1.0 / math.sqrt(hd)
        got = sc.run("mma", scale).reshape(-1, nh, hd)
        want = sc.reference(scale).reshape(-1, nh, hd)
        assert float((got.double() - want).abs().max() / want.abs().max()) < 1.2e-2
        assert float((want[-1, 0] - sc.v[0][target][0]).abs().max()) < 0.01, "the planted key does not dominate"
        assert float((got[-1, 0] - sc.v[0][target][0]).abs().max()) < 0.05, "the key that dominates was lost"


def test_a_prefetch_hint_changes_nothing():
    """The split-key kernel fetches the start of the next product's weights into L2 when asked to; the output is
    the same bit for bit, and a hint the kernel cannot use (odd strides) is dropped."""
    from flambeau_b200.kernels import ops
    sc = Scene([(700, 1), (90, 1), (1500, 2)], 8, 2, 128, 0, torch.bfloat16, seed=3)
    scale = 1.0 / math.sqrt(128)
    plain = sc.run("mma", scale)
    w = torch.randn(1024, 4096, device="cuda").bfloat16()
    assert ops.prefetch_arguments(w)[0] == w.data_ptr()
    assert torch.equal(sc.run("mma", scale, prefetch=w), plain)
    assert torch.equal(sc.run("mma", scale, prefetch=w[:, 1:]), plain)       # rows that do not start on 16 bytes
    assert ops.prefetch_arguments(w.t()) == (0, 0, 0, 0)                       # not row-major: no hint
    assert torch.equal(sc.run("mma", scale, prefetch=w.t()), plain)
    assert torch.equal(sc.run("mma", scale), plain)                            # and none stays behind


def test_hundreds_of_decoded_sequences_in_one_step():
    """Three hundred sequences at once: the split-key kernel's per-sequence arrays and its scratch grow with the step."""
    rnd = random.Random(7)
    seqs = [(rnd.randrange(0, 150), 1) for _ in range(300)]
    check(Scene(seqs, 8, 4, 64, 0, torch.bfloat16, page_size=16, seed=9), "mma")
    check(Scene(seqs[:130], 4, 4, 128, 40, torch.bfloat16, page_size=8, seed=10), "mma")


@pytest.mark.parametrize("seed", range(24))
def test_random_geometries_and_mixes(seed):
    """Seeded random scenes: head sizes in steps of 8 and 16, any grouping, page sizes that do and do not tile a
    key tile, windows, and mixes of long portions, short portions and decoded tokens, on the bfloat16 kernels."""
    rnd = random.Random(1000 + seed)
    hd = rnd.choice([16, 24, 32, 40, 48, 64, 64, 80, 96, 128, 128, 128, 160, 256])
    nkv = rnd.choice([1, 2, 3, 4, 8])
    G = rnd.choice([1, 2, 3, 4, 7, 8, 16])
    page_size = rnd.choice([8, 16, 16, 32, 64, 24, 48])
    window = rnd.choice([0, 0, 17, 64, 300])
    seqs = []
    for _ in range(rnd.randrange(1, 7)):
        kind = rnd.random()
        if kind < 0.4:
            seqs.append((rnd.randrange(0, 1200), 1))                          # a decoded token
        elif kind < 0.6:
            seqs.append((rnd.randrange(0, 600), rnd.randrange(2, 6)))         # a portion of a few tokens
        else:
            seqs.append((rnd.choice([0, 0, rnd.randrange(1, 700)]), rnd.randrange(6, 400)))   # a long portion
    if hd * nkv * G > 8192:
        nkv = 1
    check(Scene(seqs, nkv * G, nkv, hd, window, torch.bfloat16, page_size=page_size, seed=seed), "mma")


# ---- the geometry that is benchmarked: 32 query / 8 key-value heads of 128, pages of 16, a window of 4,096 --------

BENCH = dict(nh=32, nkv=8, hd=128, window=4096)


@pytest.mark.parametrize("compact", [True, False], ids=["live_rows", "rows_from_page_0"])
def test_decode_at_the_benchmarked_geometry(compact):
    """Eight decoded tokens over 8,191 cached tokens each, under the window of 4,096: the leading 255 pages of each
    sequence are given back (and, in the engine's form of the table, not in the row at all)."""
    sc = Scene([(8191, 1)] * 8, dtype=torch.bfloat16, seed=21, compact=compact, **BENCH)
    if compact:
        assert int(sc.table_base[0]) == (8191 - 4096 + 1) // 16 == 256 and sc.table.shape[1] < 8192 // 16
    check(sc, "mma")


def test_decode_mix_at_the_benchmarked_geometry():
    """Twenty-four decoded tokens with contexts between 4,000 and 8,191 tokens under the window of 4,096."""
    rnd = random.Random(5)
    seqs = [(rnd.randrange(4000, 8192), 1) for _ in range(23)] + [(8191, 1)]
    check(Scene(seqs, dtype=torch.bfloat16, seed=22, compact=True, **BENCH), "mma")


def test_a_far_key_at_the_benchmarked_geometry():
    """Over 8,191 cached tokens one key is made to dominate: the first key the window still shows is found, the key
    just before it is not."""
    nh, nkv, hd, window = BENCH["nh"], BENCH["nkv"], BENCH["hd"], BENCH["window"]
    p = 8191
    for target, seen in ((p - window + 1, True), (p - window, False), (6000, True)):
        sc = Scene([(p, 1), (5000, 1)], dtype=torch.bfloat16, seed=target, spread=0.3, compact=True, **BENCH)
        for h in range(nkv):
            qh = sc.q[0][0, h * (nh // nkv)]
            sc.k[0][target, h] = (qh / qh.norm() * 60.0).to(torch.bfloat16).float()
        pid = sc.page_of(0, target)
        if pid >= 0:
            sc.k_pool[pid, :, target % 16] = sc.k[0][target]
        scale = 1.0 / math.sqrt(hd)
        got = sc.run("mma", scale).reshape(-1, nh, hd)
        want = sc.reference(scale).reshape(-1, nh, hd)
        assert float((got.double() - want).abs().max() / want.abs().max()) < 1.2e-2
        close = float((got[0, 0] - sc.v[0][target][0]).abs().max())
        assert (close < 0.05) if seen else (close > 0.3)


@pytest.mark.parametrize("cached", [0, 6000])
def test_a_2048_token_portion_at_the_benchmarked_geometry(prompt_kernel, cached):
    """A portion of 2,048 tokens from position 0, and from position 6,000 where every query's window has left the
    start of the cache behind."""
    sc = Scene([(cached, 2048)], dtype=torch.bfloat16, seed=23 + cached, compact=True, **BENCH)
    check(sc, "mma")
