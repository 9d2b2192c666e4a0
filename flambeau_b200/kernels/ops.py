"""Tensor-level wrappers of the kernel launchers.

Each wrapper checks devices, dtypes and strides, then launches on torch's
current CUDA stream.  Constants (eps, theta-derived tables, head sizes, window,
scale) arrive as arguments; nothing here knows a model.
"""
from __future__ import annotations

import ctypes

import torch

from .library import KernelError, check, lib

_CODES = {torch.float32: 0, torch.bfloat16: 1}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 or bfloat16)") from None


try:                                   # the raw handle of torch's current stream, without building a Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:                 # a torch without it: the public way, a few microseconds slower per launch
    _raw_stream = None


def current_stream() -> int:
    """The CUDA stream the kernels are queued on: torch's current stream of the current device."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_stream = current_stream


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on the GPU; there is no CPU path")


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _rows(t: torch.Tensor) -> int:
    """Row stride (elements) of a 2-d tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"expected a 2-d tensor with dense rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def _i32(t, what):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32")


# ---------------------------------------------------------------------------

def embedding(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor, status: torch.Tensor) -> None:
    _cuda(table, ids, x, status)
    _i32(ids, "token ids")
    V, H = table.shape
    n = ids.numel()
    if x.dtype != torch.float32 or x.shape[0] < n or x.shape[1] != H or not x.is_contiguous() \
            or not table.is_contiguous():
        raise KernelError("embedding: the stream must be contiguous float32 [n, width]")
    check(lib().fb_embedding(table.data_ptr(), dtype_code(table), ids.data_ptr(), x.data_ptr(), n, H, V,
                             status.data_ptr(), _stream()), "embedding")


def add_rms_norm(x: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor,
                 rows=None, n_partials: int = 1, n_rows: int | None = None, partial_stride: int = 0,
                 weight_offset: float = 0.0) -> None:
    """out[j] = rmsnorm(x[r] + sum_p delta_p[r]) * (weight + weight_offset), r = rows[j] or j; without `rows`
    the sum is also written back to x.  `delta` is [n, H]; with n_partials > 1 it is the first of that many
    slabs `partial_stride` elements apart.  weight_offset is 0 for a plain weight, 1 for a "1 + w" norm."""
    _cuda(x, delta, weight, out, rows)
    _i32(rows, "rows")
    H = x.shape[1]
    n_out = rows.numel() if rows is not None else (x.shape[0] if n_rows is None else n_rows)
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or out.shape[-1] != H \
            or weight.numel() != H or out.shape[0] < n_out:
        raise KernelError("add_rms_norm: bad shapes")
    stride = 0
    if delta is not None:
        if not delta.is_contiguous() or delta.shape[-1] != H:
            raise KernelError("add_rms_norm: delta must be contiguous with the stream's width")
        if n_partials > 1:
            stride = int(partial_stride)
            if stride <= 0:
                raise KernelError("add_rms_norm: several slabs need their stride")
    check(lib().fb_add_rmsnorm(x.data_ptr(), _ptr(delta), dtype_code(delta) if delta is not None else 0,
                               n_partials, stride, weight.data_ptr(), dtype_code(weight), out.data_ptr(),
                               dtype_code(out), _ptr(rows), n_out, H, float(eps), float(weight_offset), _stream()),
          "add_rms_norm")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    _cuda(positions, inv_freq, cos, sin)
    _i32(positions, "positions")
    n, half = positions.numel(), inv_freq.numel()
    if inv_freq.dtype != torch.float64 or cos.dtype != torch.float32 or sin.dtype != torch.float32 \
            or cos.numel() < n * half or sin.numel() < n * half:
        raise KernelError("rope_table: bad arguments")
    check(lib().fb_rope_table(positions.data_ptr(), inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), n, half,
                              _stream()), "rope_table")


def rope_kv_write(q_in, q_out, k, v, cos, sin, half: int, positions, row_seq, block_table, k_pool, v_pool,
                  page_size: int, nh: int, nkv: int, hd: int, write_kv: bool, status, n_partials: int = 1,
                  partial_stride: int = 0, table_base=None) -> None:
    """q_out = rotate(q_in) (q_out may be q_in); with write_kv, rotate k into the cache and copy v into it.
    q_in, k, v share one dtype (the projection's output); q_out and the cache share one dtype.  With
    n_partials > 1 the inputs are split-K shares `partial_stride` elements apart and are added first.
    table_base (int32 per sequence, optional): the logical page that column 0 of each table row stands for."""
    _cuda(q_in, q_out, k, v, cos, sin, positions, row_seq, block_table, k_pool, v_pool, status, table_base)
    _i32(table_base, "table_base")
    n = q_in.shape[0]
    if q_in.shape[1] != nh * hd or q_out.shape[1] != nh * hd or q_out.shape[0] != n:
        raise KernelError("rope_kv_write: q widths do not match the head counts")
    if write_kv:
        if k.shape[1] != nkv * hd or v.shape[1] != nkv * hd:
            raise KernelError("rope_kv_write: k/v widths do not match the head counts")
        if k.dtype != q_in.dtype or v.dtype != q_in.dtype or k_pool.dtype != q_out.dtype or v_pool.dtype != q_out.dtype:
            raise KernelError("rope_kv_write: inputs must share one dtype; q_out and the cache another")
    n_pages = k_pool.shape[0] if write_kv else 0
    if write_kv and (tuple(k_pool.shape) != (n_pages, nkv, page_size, hd) or not k_pool.is_contiguous()
                     or tuple(v_pool.shape) != tuple(k_pool.shape) or not v_pool.is_contiguous()):
        raise KernelError("rope_kv_write: cache pools must be contiguous [pages, kv heads, page size, head size]")
    check(lib().fb_rope_kv_write(
        q_in.data_ptr(), _rows(q_in), int(n_partials), int(partial_stride), q_out.data_ptr(), _rows(q_out), _ptr(k),
        _rows(k) if k is not None else 0,
        _ptr(v), _rows(v) if v is not None else 0, dtype_code(q_in), dtype_code(q_out), _ptr(cos), _ptr(sin), half,
        _ptr(positions), _ptr(row_seq), _ptr(block_table),
        block_table.stride(0) if block_table is not None else 0, _ptr(table_base), _ptr(k_pool), _ptr(v_pool),
        page_size, n_pages, n, nh, nkv if write_kv else 0, hd, 1 if write_kv else 0, status.data_ptr(), _stream()),
        "rope_kv_write")


ACTIVATIONS = {"silu": 1, "gelu_tanh": 2, "gelu_pytorch_tanh": 2}      # codes of the kernels' gate activations


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation '{name}' is not implemented; known: {', '.join(sorted(ACTIVATIONS))}") from None


def gate_mul(gate_up: torch.Tensor, out: torch.Tensor, n_partials: int = 1, partial_stride: int = 0,
             activation: str = "silu") -> None:
    """out[:, c] = act(gate_up[:, 2c]) * gate_up[:, 2c+1] (gate and up alternate along a row); with
    n_partials > 1, gate_up is the first of that many split-K shares `partial_stride` elements apart, which are
    added first."""
    _cuda(gate_up, out)
    n, two_i = gate_up.shape
    I = two_i // 2
    if tuple(out.shape) != (n, I) or not out.is_contiguous():
        raise KernelError("gate_mul: bad output")
    check(lib().fb_gate_mul(gate_up.data_ptr(), _rows(gate_up), dtype_code(gate_up), int(n_partials),
                            int(partial_stride), out.data_ptr(), dtype_code(out), n, I, activation_code(activation),
                            _stream()), "gate_mul")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, n_partials: int = 1, partial_stride: int = 0) -> None:
    gate_mul(gate_up, out, n_partials, partial_stride, "silu")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T, float32 accumulation on the CUDA cores."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    check(lib().fb_gemm_simt(a.data_ptr(), dtype_code(a), _rows(a), w.data_ptr(), dtype_code(w), _rows(w),
                             out.data_ptr(), dtype_code(out), _rows(out), M, N, K, _stream()), "gemm_simt", (M, N, K))


def _slopes(score_slopes, nh: int) -> int:
    """The address of the per-head slopes (float32 [nh], contiguous, on the GPU), or 0 for none."""
    if score_slopes is None:
        return 0
    if not score_slopes.is_cuda or score_slopes.dtype != torch.float32 or score_slopes.numel() != nh \
            or not score_slopes.is_contiguous():
        raise KernelError(f"attention: score slopes must be {nh} contiguous float32 on the GPU, one per query head")
    return score_slopes.data_ptr()


def paged_attention_simt(q, out, k_pool, v_pool, block_table, positions, row_seq, nh: int, nkv: int, hd: int,
                         window: int, scale: float, status, table_base=None, score_slopes=None) -> None:
    """score_slopes (float32 per query head, optional): slope * (key position - query position) is added to every
    scaled score, a linear penalty on distance."""
    _cuda(q, out, k_pool, v_pool, block_table, positions, row_seq, status, table_base)
    _i32(table_base, "table_base")
    n = q.shape[0]
    n_pages, pool_kv, page_size, pool_hd = k_pool.shape
    if pool_kv != nkv or pool_hd != hd or q.shape[1] != nh * hd or out.shape[1] != nh * hd or out.shape[0] != n:
        raise KernelError("attention: shapes do not match the head counts")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype):
        raise KernelError("attention: q, out and the cache must share one dtype")
    if not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("attention: cache pools must be contiguous")
    check(lib().fb_paged_attention_simt(
        q.data_ptr(), _rows(q), out.data_ptr(), _rows(out), dtype_code(q), k_pool.data_ptr(), v_pool.data_ptr(),
        page_size, n_pages, block_table.data_ptr(), block_table.stride(0), _ptr(table_base), positions.data_ptr(),
        row_seq.data_ptr(), n, nh, nkv, hd, int(window), float(scale), _slopes(score_slopes, nh), status.data_ptr(),
        _stream()), "paged_attention_simt")


def apply_penalties(logits, rows, tokens, counts, repetition, presence, frequency) -> None:
    _cuda(logits, rows, tokens, counts, repetition, presence, frequency)
    check(lib().fb_apply_penalties(logits.data_ptr(), _rows(logits), logits.shape[1], rows.data_ptr(),
                                   tokens.data_ptr(), counts.data_ptr(), repetition.data_ptr(),
                                   presence.data_ptr(), frequency.data_ptr(), rows.numel(), _stream()),
          "apply_penalties")


def apply_logit_bias(logits, rows, tokens, bias) -> None:
    _cuda(logits, rows, tokens, bias)
    check(lib().fb_apply_logit_bias(logits.data_ptr(), _rows(logits), logits.shape[1], rows.data_ptr(),
                                    tokens.data_ptr(), bias.data_ptr(), rows.numel(), _stream()),
          "apply_logit_bias")


def sample(logits, out, temperature=None, uniform=None, top_k=None, top_p=None, min_p=None, n=None) -> None:
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or no temperature given), else a draw."""
    _cuda(logits, out, temperature, uniform, top_k, top_p, min_p)
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    _i32(out, "sampled tokens")
    _i32(top_k, "top_k")
    n = logits.shape[0] if n is None else n
    check(lib().fb_sample(logits.data_ptr(), _rows(logits), n, logits.shape[1], _ptr(temperature), _ptr(uniform),
                          _ptr(top_k), _ptr(top_p), _ptr(min_p), out.data_ptr(), _stream()), "sample")


# ---------------------------------------------------------------------------
# choices between kernels of one family
# ---------------------------------------------------------------------------

class _SplitScratch:
    """Float32 partial tiles and per-tile arrival counters of the split-K tensor-core product, per device.
    Kernels of one stream run in order, so one buffer serves every product of the step."""
    PARTIAL_FLOATS = 16 << 20
    COUNTERS = 8192
    _by_device: dict = {}

    @classmethod
    def get(cls, device):
        hit = cls._by_device.get(device)
        if hit is None:
            hit = (torch.empty(cls.PARTIAL_FLOATS, dtype=torch.float32, device=device),
                   torch.zeros(cls.COUNTERS, dtype=torch.int32, device=device))
            cls._by_device[device] = hit
        return hit


def tc_supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands: bfloat16, 16-byte aligned, row strides of 8 elements."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in _CODES
            and a.dim() == 2 and w.dim() == 2 and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_SPLITS_USED = ctypes.c_int(1)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor, splits: int = 0,
            slabs: torch.Tensor | None = None) -> int:
    """out[M,N] = a[M,K] @ w[N,K]^T on the tensor cores (bfloat16 operands, float32 accumulation).
    splits = 0 lets the launcher choose the split of K.  With `slabs` (float32 [P, M, N], out = slabs[0]) each
    split writes its share into its own slab and the count of slabs to add is returned; otherwise the kernel
    adds the shares itself and 1 is returned."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: operands must be bfloat16")
    slab_stride = max_slabs = 0
    if slabs is not None:
        if slabs.dtype != torch.float32 or slabs.dim() != 3 or slabs.data_ptr() != out.data_ptr():
            raise KernelError("gemm_tc: slabs must be float32 [P, M, N] with out = slabs[0]")
        slab_stride, max_slabs = slabs.stride(0), slabs.shape[0]
    partials, counters = _SplitScratch.get(a.device)
    check(lib().fb_gemm_tc(a.data_ptr(), _rows(a), w.data_ptr(), _rows(w), out.data_ptr(), dtype_code(out),
                           _rows(out), slab_stride, max_slabs, ctypes.byref(_SPLITS_USED), M, N, K,
                           partials.data_ptr(), partials.numel(), counters.data_ptr(), counters.numel(),
                           int(splits), status.data_ptr(), _stream()), "gemm_tc", (M, N, K))
    return _SPLITS_USED.value if slabs is not None else 1


def gemm_tc_add(a: torch.Tensor, w: torch.Tensor, acc: torch.Tensor, status: torch.Tensor, max_slabs: int = 1) -> bool:
    """acc[M,N] += a[M,K] @ w[N,K]^T in float32, where the product is one the two-SM tensor-core kernel takes in
    whole tiles (hundreds of rows, and no split of K would be chosen although `max_slabs` slabs could be had): each
    element of acc gets one float32 add from the kernel's epilogue.  Returns False, having done nothing, for any
    other product: the caller then leaves the output where another kernel adds it."""
    _cuda(a, w, acc, status)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or acc.shape[0] < M or acc.shape[1] != N:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} acc{tuple(acc.shape)} do not agree")
    if acc.dtype != torch.float32 or not tc_supported(a, w, acc) or M <= 128:
        return False
    rc = lib().fb_gemm_tc_add(a.data_ptr(), _rows(a), w.data_ptr(), _rows(w), acc.data_ptr(), _rows(acc),
                              int(max_slabs), M, N, K, status.data_ptr(), _stream())
    if rc == 0:
        return False                         # nothing was launched
    check(0 if rc == 1 else rc, "gemm_tc_add", (M, N, K))
    return True


def gemm_tc_gated(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
                  activation: str = "silu") -> None:
    """out[M, N/2] = act(g) * u where (g_0, u_0, g_1, u_1, ...) = a @ w^T: w stacks gate and up rows alternately
    and the activation runs in the product's epilogue."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] * 2 != N:
        raise KernelError(f"gated gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    partials, counters = _SplitScratch.get(a.device)
    check(lib().fb_gemm_tc_gated(a.data_ptr(), _rows(a), w.data_ptr(), _rows(w), out.data_ptr(), dtype_code(out),
                                 _rows(out), M, N, K, activation_code(activation), partials.data_ptr(),
                                 partials.numel(), counters.data_ptr(), counters.numel(), status.data_ptr(),
                                 _stream()), "gemm_tc_gated", (M, N, K))


def linear_slabs(a: torch.Tensor, w: torch.Tensor, slabs: torch.Tensor, ctx) -> int:
    """slabs[0] + ... + slabs[k-1] = a @ w^T; returns k.  The tensor-core kernel leaves the split-K shares for the
    next kernel to add; every other path writes the whole product into slabs[0]."""
    out = slabs[0]
    if slabs.shape[0] > 1 and tc_supported(a, w, out):
        return gemm_tc(a, w, out, ctx.runtime.status, slabs=slabs)
    linear(a, w, out, ctx)
    return 1


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ctx=None) -> None:
    """out = a @ w^T with the kernel that fits the dtypes and the shape: the tcgen05 kernel for bfloat16
    operands it can fetch by TMA, the float32-FMA kernel for everything else (all of the 32-bit mode)."""
    if ctx is not None and tc_supported(a, w, out):
        gemm_tc(a, w, out, ctx.runtime.status)
    else:
        gemm_simt(a, w, out)


class _AttentionScratch:
    """Float32 partial outputs of the split-key attention arrangement and its per-pair arrival counters, per
    device.  The counters must be zero between launches: the kernel leaves them so.  The buffer grows with the
    largest step seen; outgrown buffers stay alive because captured graphs may hold their addresses."""
    _by_device: dict = {}
    _outgrown: list = []

    @classmethod
    def get(cls, device, n_seqs: int, nkv: int, hd: int):
        hd_max = 32 if hd <= 32 else 64 if hd <= 64 else 128 if hd <= 128 else 256
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        pairs = n_seqs * nkv
        # 65536 counters, then one partial per slot: at most 4 resident CTAs per SM plus one slot per pair
        need = (1 << 16) + (4 * sms + pairs) * (16 * hd_max + 32)
        hit = cls._by_device.get(device)
        if hit is None or hit.numel() < need:
            if hit is not None:
                cls._outgrown.append(hit)
            floats = max(1 << 22, 1 << (need - 1).bit_length())
            hit = cls._by_device[device] = torch.zeros(floats, dtype=torch.float32, device=device)
        return hit


def prefetch_arguments(weight, budget_bytes: int = 16 << 20) -> tuple:
    """(base, rows, row stride in bytes, bytes per row) for the attention launcher's L2 hint: the first bytes of
    every row of `weight` ([rows, K], the matrix of the product that follows), `budget_bytes` in all, which the
    split-key kernel fetches into L2 when its stream of cache ends, so that the product starts on data that is
    already on the chip.  A hint: results do not depend on it; a matrix the kernel cannot take gives no hint.
    (Measured for the row-wise kernels between the products and for the products' own tails as well: there it
    costs more than it brings.)"""
    if weight is None or weight.dim() != 2 or weight.stride(1) != 1:
        return (0, 0, 0, 0)
    rows = weight.shape[0]
    row_bytes = weight.shape[1] * weight.element_size()
    per_row = min(row_bytes, max(512, (budget_bytes // max(rows, 1)) // 512 * 512)) // 16 * 16
    if per_row < 16:
        return (0, 0, 0, 0)
    return (weight.data_ptr(), rows, weight.stride(0) * weight.element_size(), per_row)


def set_gemm_pair(on: bool) -> None:
    """Products with hundreds of rows on the two-SM kernel (tcgen05 cta_group::2) where there are enough tiles
    (the default), or always on the one-SM kernel."""
    lib().fb_set_gemm_pair(1 if on else 0)


def set_attention_tc(on: bool) -> None:
    """Portions of prompts on the tcgen05 attention kernel where it takes the geometry (the default), or always on
    the mma.sync kernel."""
    lib().fb_set_attention_tc(1 if on else 0)


def mma_attention_supported(q: torch.Tensor, nh: int, nkv: int, hd: int) -> bool:
    return (q.dtype == torch.bfloat16 and hd % 8 == 0 and hd <= 256 and nh % nkv == 0 and nh // nkv <= 64
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def paged_attention_mma(q, out, k_pool, v_pool, block_table, seq_q_start, seq_q_len, seq_pos_start, n_seqs: int,
                        max_q_len: int, max_kv_len: int, any_short: bool, any_long: bool, nh: int, nkv: int,
                        hd: int, window: int, scale: float, status, table_base=None, prefetch=None,
                        multi_seqs=None, n_multi: int = 0, score_slopes=None) -> None:
    """bfloat16 attention on the tensor cores over the paged cache; sequences are described per entry of the
    step (first row, rows, first position).  any_short / any_long say whether the step holds sequences with
    rows * (nh/nkv) <= 16 / > 16, which run in different arrangements of the kernel.  table_base (int32 per
    sequence, optional): the logical page that column 0 of each table row stands for.  prefetch (optional): the
    weight matrix of the product that follows (see prefetch_arguments).  multi_seqs (int32, optional): the
    n_multi sequences of the step that bring more than one token; the kernels for portions then lay their grid over
    these instead of over every sequence.  score_slopes (float32 per query head, optional): slope * (key position -
    query position) is added to every scaled score; portions then run on the mma.sync kernel."""
    _cuda(q, out, k_pool, v_pool, block_table, seq_q_start, seq_q_len, seq_pos_start, status, table_base, multi_seqs)
    _i32(table_base, "table_base")
    _i32(multi_seqs, "multi_seqs")
    n_pages, pool_kv, page_size, pool_hd = k_pool.shape
    if pool_kv != nkv or pool_hd != hd or q.shape[1] != nh * hd or out.shape[1] != nh * hd:
        raise KernelError("attention: shapes do not match the head counts")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16):
        raise KernelError("attention_mma: q, out and the cache must be bfloat16")
    if not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("attention: cache pools must be contiguous")
    scratch = _AttentionScratch.get(q.device, n_seqs, nkv, hd)
    check(lib().fb_paged_attention_mma(
        q.data_ptr(), _rows(q), out.data_ptr(), _rows(out), k_pool.data_ptr(), v_pool.data_ptr(), page_size, n_pages,
        block_table.data_ptr(), block_table.stride(0), _ptr(table_base), seq_q_start.data_ptr(),
        seq_q_len.data_ptr(), seq_pos_start.data_ptr(), _ptr(multi_seqs), int(n_multi), n_seqs, max_q_len, max_kv_len,
        1 if any_short else 0,
        1 if any_long else 0, nh, nkv, hd, int(window), float(scale), _slopes(score_slopes, nh), scratch.data_ptr(),
        scratch.numel(),
        *prefetch_arguments(prefetch), status.data_ptr(), _stream()), "paged_attention_mma")


def paged_attention(ctx, q, out, cache, nh: int, nkv: int, hd: int, window: int, scale: float,
                    next_weight=None, score_slopes=None) -> None:
    """Attention of every row of the step over its request's cached keys: the tensor-core kernel for bfloat16
    and head sizes it takes, the float32 CUDA-core kernel otherwise (all of the 32-bit mode).  next_weight: the
    matrix of the product that follows, whose start the bfloat16 kernel may fetch into L2 (a hint)."""
    b = ctx.batch
    if mma_attention_supported(q, nh, nkv, hd):
        G = nh // nkv
        short = [ql * G <= 16 for ql in b.seq_q_len]
        paged_attention_mma(q, out, cache.k_pool, cache.v_pool, cache.block_table, b.seq_q_start_d, b.seq_q_len_d,
                            b.seq_pos_start_d, b.n_seqs, b.max_q_len, b.max_kv_len, any(short), not all(short),
                            nh, nkv, hd, window, scale, ctx.runtime.status, table_base=cache.table_base,
                            prefetch=next_weight, multi_seqs=b.multi_seqs_d, n_multi=b.n_multi,
                            score_slopes=score_slopes)
    else:
        paged_attention_simt(q, out, cache.k_pool, cache.v_pool, cache.block_table, b.positions, b.row_seq,
                             nh, nkv, hd, window, scale, ctx.runtime.status, table_base=cache.table_base,
                             score_slopes=score_slopes)
