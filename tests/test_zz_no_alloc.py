"""The entry point that allocates nothing (csrc/no_alloc.h), called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need a product: a host program that
gave all device memory to its own pool at start-up, or a serving loop that cannot afford the device-wide
synchronisation that cudaMalloc and cudaFree bring.  For them fb_gemm_tc_noalloc runs the split-K tensor-core
product with its scratch in a fixed array inside the library.  This test calls it twice in a row, with different
operands, compares each result with the ordinary entry point's, checks that the free device memory did not move,
and checks that sizes beyond the stated maximum are refused.  It runs last so that a failure here cannot hide
another test's result; it must pass alone in a fresh process as well as after all the others.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def load():
    from flambeau_b200.kernels.library import library_path
    handle = ctypes.CDLL(library_path())
    fn = handle.fb_gemm_tc_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                   ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p]
    handle.fb_last_error.restype = ctypes.c_char_p
    return handle, fn


def call(fn, x, w, out, status):
    code = {torch.float32: 0, torch.bfloat16: 1}[out.dtype]
    return fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), code, out.stride(0),
              x.shape[0], w.shape[0], x.shape[1], status.data_ptr(), torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,N,K,out_dtype", [(8, 4096, 4096, torch.float32), (1, 1000, 14336, torch.float32),
                                             (64, 6144, 4096, torch.bfloat16), (33, 130, 72, torch.float32)])
def test_two_calls_in_a_row_match_the_ordinary_entry_point(M, N, K, out_dtype):
    from flambeau_b200.kernels import ops
    handle, fn = load()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    operands = []
    for _ in range(2):
        x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        w = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
        want = torch.empty(M, N, device="cuda", dtype=out_dtype)
        ops.gemm_tc(x, w, want, status)                       # the existing entry point, scratch from the caller
        operands.append((x, w, want, torch.full((M, N), float("nan"), device="cuda", dtype=out_dtype)))
    torch.cuda.synchronize()
    # the first call on the device may do its one-time set-up; the second must not move the free memory
    assert call(fn, *operands[0][:2], operands[0][3], status) == 0, handle.fb_last_error().decode()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert call(fn, *operands[1][:2], operands[1][3], status) == 0, handle.fb_last_error().decode()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the call allocated or freed device memory"
    assert int(status.item()) == 0
    tol = 2e-5 if out_dtype == torch.float32 else 8e-3       # the tolerances of the product's own tests
    for x, w, want, got in operands:
        assert torch.isfinite(got).all()
        err = float((got.double() - want.double()).abs().max() / want.double().abs().max())
        assert err < tol, f"differs from the ordinary entry point by {err:.2e}"
        exact = x.double() @ w.double().T
        assert float((got.double() - exact).abs().max() / exact.abs().max()) < tol


def test_sizes_beyond_the_maximum_are_refused_with_a_message():
    handle, fn = load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.zeros(65, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(65, 128, device="cuda")
    assert call(fn, x, w, out, status) != 0
    msg = handle.fb_last_error().decode()
    assert "65 rows exceed the maximum of 64" in msg
    x = torch.zeros(2, 72, device="cuda", dtype=torch.bfloat16)[:, :70]       # row stride 72, K = 70: fine
    w = torch.zeros(8, 20, device="cuda", dtype=torch.bfloat16)               # row stride 20: not a multiple of 8
    assert call(fn, x[:, :20], w, torch.zeros(2, 8, device="cuda"), status) != 0
    assert "multiples of 8" in handle.fb_last_error().decode()
