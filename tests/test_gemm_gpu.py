"""The matrix-product kernels alone against torch's float32/float64 product, at sizes other than the engine's."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    return float((got.double() - want).abs().max() / want.abs().max())


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 96), (17, 64, 160), (70, 321, 64), (300, 257, 100), (5, 1000, 24)])
@pytest.mark.parametrize("dt", ["fff", "bbf", "bbb", "bff"])
def test_simt_product(M, N, K, dt):
    from flambeau_b200.kernels import ops
    t = {"f": torch.float32, "b": torch.bfloat16}
    g = torch.Generator(device="cuda").manual_seed(M * 1000 + N)
    a = torch.randn(M, K, device="cuda", generator=g).to(t[dt[0]])
    w = torch.randn(N, K, device="cuda", generator=g).to(t[dt[1]])
    wide = torch.zeros(M, N + 3, device="cuda", dtype=t[dt[2]])
    out = wide[:, :N]                                    # a strided output
    ops.gemm_simt(a, w, out)
    want = a.double() @ w.double().T
    tol = 1e-5 if dt[2] == "f" else 8e-3
    assert rel_err(out, want) < tol
    assert float(wide[:, N:].abs().max()) == 0.0


SHAPES_TC = [
    (1, 128, 64), (8, 256, 512), (8, 6144, 4096), (16, 384, 1024), (17, 130, 72), (33, 4096, 4096),
    (64, 1000, 264), (65, 257, 8), (128, 512, 2048), (200, 320, 96), (256, 1024, 1024), (300, 200, 136),
    (515, 4096, 1024), (2048, 1024, 4096),
    # enough tiles of 256 x 256 for every pair of SMs: the two-SM kernel
    (300, 10000, 200), (700, 6500, 1000), (2048, 4096, 4096), (515, 20000, 64), (129, 19000, 72),
]


@pytest.mark.parametrize("M,N,K", SHAPES_TC)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_tensor_core_product(M, N, K, out_dtype, splits):
    from flambeau_b200.kernels import ops
    if splits > (K + 63) // 64:
        pytest.skip("more splits than 64-wide blocks of K")
    g = torch.Generator(device="cuda").manual_seed(M + 7 * N + 13 * K)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((M, N), float("nan"), device="cuda", dtype=out_dtype)
    assert ops.tc_supported(a, w, out)
    ops.gemm_tc(a, w, out, status, splits=splits)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
    want = a.double() @ w.double().T
    assert torch.isfinite(out).all()
    tol = 2e-5 if out_dtype == torch.float32 else 8e-3
    assert rel_err(out, want) < tol
    # twice in a row: the split-K counters must have been left at zero
    out2 = torch.empty_like(out)
    ops.gemm_tc(a, w, out2, status, splits=splits)
    assert torch.equal(out, out2), "the product is not reproducible"


@pytest.mark.parametrize("M,N,K", [(300, 10000, 200), (2048, 6144, 1024), (1000, 9999, 136), (257, 1024, 128),
                                   (536, 3000, 264), (1056, 2048, 512), (400, 4100, 72), (2080, 1536, 256)])
def test_two_sm_product_equals_the_one_sm_product(M, N, K):
    """Both kernels add the same products in the same order, so they agree to the bit.  Row counts that leave a
    last token tile of 1, 24, 32, 44, 144 and 232 rows: the two-SM kernel multiplies that tile at its own width."""
    from flambeau_b200.kernels import ops
    g = torch.Generator(device="cuda").manual_seed(M + N)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = []
    try:
        for pair in (True, False):
            ops.set_gemm_pair(pair)
            out = torch.full((M, N), float("nan"), device="cuda")
            ops.gemm_tc(a, w, out, status, splits=1)           # one share of K in both: the same order of sums
            outs.append(out)
    finally:
        ops.set_gemm_pair(True)
    assert int(status.item()) == 0
    assert torch.equal(outs[0], outs[1])
    assert rel_err(outs[0], a.double() @ w.double().T) < 2e-5


@pytest.mark.parametrize("M,N,K,taken", [(2048, 4096, 4096, True), (2048, 4096, 14336, True), (600, 5000, 264, True),
                                         (2080, 1536, 520, True), (257, 10000, 128, True), (64, 4096, 4096, False),
                                         (128, 1024, 512, False), (512, 1024, 16384, False)])
def test_product_added_to_its_output(M, N, K, taken):
    """acc += a w^T from the two-SM kernel's epilogue: one float32 add per element, edges of the output clipped,
    twice in a row for the second add, reproducible; and products that the kernel does not take in whole tiles (few
    rows; a long K on few tiles, which wants shares) are declined with the output untouched."""
    from flambeau_b200.kernels import ops
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc0 = torch.randn(M + 3, N, device="cuda", generator=g)           # rows beyond M belong to someone else
    acc = acc0.clone()
    assert ops.gemm_tc_add(a, w, acc, status, max_slabs=4) == taken
    if not taken:
        assert torch.equal(acc, acc0)
        return
    exact = a.double() @ w.double().T
    assert int(status.item()) == 0
    assert torch.equal(acc[M:], acc0[M:])
    assert rel_err(acc[:M], acc0[:M].double() + exact) < 2e-5
    again = acc0.clone()
    assert ops.gemm_tc_add(a, w, again, status, max_slabs=4)
    assert torch.equal(acc, again), "the sum is not reproducible"
    assert ops.gemm_tc_add(a, w, acc, status, max_slabs=4)
    assert rel_err(acc[:M], acc0[:M].double() + 2 * exact) < 2e-5
    # an output whose rows are not 16 bytes apart has no tensor map: the warps add for themselves
    wide = torch.randn(M, N + 1, device="cuda", generator=g)
    view0 = wide[:, :N].clone()
    assert ops.gemm_tc_add(a, w, wide[:, :N], status, max_slabs=4)
    assert rel_err(wide[:, :N], view0.double() + exact) < 2e-5 and int(status.item()) == 0


@pytest.mark.parametrize("M,N,K,P", [(8, 4096, 4096, 16), (64, 512, 8192, 8), (40, 1000, 264, 4), (512, 4096, 14336, 8),
                                     (300, 1000, 8192, 4), (1024, 2048, 4096, 8), (2048, 4096, 1024, 4)])
def test_shares_of_k_left_in_slabs(M, N, K, P):
    """With slabs the kernel leaves its split-K shares for the consumer to add: k slabs hold the product,
    the others are untouched."""
    from flambeau_b200.kernels import ops
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    slabs = torch.full((P, M, N), float("nan"), device="cuda")
    k = ops.gemm_tc(a, w, slabs[0], status, slabs=slabs)
    assert 1 <= k <= P and int(status.item()) == 0
    assert torch.isfinite(slabs[:k]).all() and torch.isnan(slabs[k:]).all()
    assert rel_err(slabs[:k].double().sum(0), a.double() @ w.double().T) < 2e-5
    again = torch.full((P, M, N), float("nan"), device="cuda")
    assert ops.gemm_tc(a, w, again[0], status, slabs=again) == k
    assert torch.equal(slabs[:k], again[:k])


def test_tensor_core_product_on_strided_views():
    from flambeau_b200.kernels import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    big_a = torch.randn(40, 200, device="cuda", generator=g).to(torch.bfloat16)
    big_w = torch.randn(300, 200, device="cuda", generator=g).to(torch.bfloat16)
    a, w = big_a[:, 8:136], big_w[:, 64:192]               # 16-byte aligned column offsets, K = 128
    wide = torch.zeros(40, 304, device="cuda", dtype=torch.float32)
    out = wide[:, :300]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert ops.tc_supported(a, w, out)
    ops.gemm_tc(a, w, out, status)
    assert rel_err(out, a.double() @ w.double().T) < 2e-5
    assert float(wide[:, 300:].abs().max()) == 0.0 and int(status.item()) == 0


def test_shapes_the_tma_path_cannot_take_are_refused():
    from flambeau_b200.kernels import ops
    from flambeau_b200.kernels.library import KernelError
    a = torch.zeros(4, 20, device="cuda", dtype=torch.bfloat16)    # row stride 20 elements = 40 bytes
    w = torch.zeros(8, 20, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(4, 8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert not ops.tc_supported(a, w, out)
    with pytest.raises(KernelError):
        ops.gemm_tc(a, w, out, status)
    with pytest.raises(KernelError):
        ops.gemm_tc(a.float(), w, out, status)


@pytest.mark.parametrize("M,I,K", [(3, 64, 64), (17, 100, 136), (70, 1001, 72), (300, 160, 96), (2048, 512, 256),
                                   (600, 4001, 136), (2048, 2560, 256)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gated_epilogue(M, I, K, out_dtype):
    """Gate and up rows alternate in the weight; the epilogue writes silu(gate) * up, half as wide."""
    from flambeau_b200.kernels import ops
    g = torch.Generator(device="cuda").manual_seed(M + I)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda", generator=g) / 8).to(torch.bfloat16)
    out = torch.full((M, I), float("nan"), device="cuda", dtype=out_dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemm_tc_gated(a, w, out, status)
    y = a.double() @ w.double().T
    gate, up = y[:, 0::2], y[:, 1::2]
    want = gate / (1 + torch.exp(-gate)) * up
    assert int(status.item()) == 0 and torch.isfinite(out).all()
    assert rel_err(out, want) < (3e-5 if out_dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("M,I,K", [(5, 100, 136), (300, 160, 96), (1056, 512, 256)])
def test_gated_epilogue_with_another_activation(M, I, K):
    """The activation of the epilogue is an argument: gelu (tanh form) beside silu, in the one-SM and the two-SM kernel."""
    import math
    from flambeau_b200.kernels import ops
    g = torch.Generator(device="cuda").manual_seed(M + I)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda", generator=g) / 8).to(torch.bfloat16)
    out = torch.full((M, I), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemm_tc_gated(a, w, out, status, activation="gelu_tanh")
    y = a.double() @ w.double().T
    gate, up = y[:, 0::2], y[:, 1::2]
    want = 0.5 * gate * (1 + torch.tanh(math.sqrt(2 / math.pi) * (gate + 0.044715 * gate ** 3))) * up
    assert int(status.item()) == 0 and torch.isfinite(out).all()
    assert rel_err(out, want) < 3e-5
