"""Loads the compiled kernel library and declares the C signatures.

There is no fallback: if the library cannot be built or loaded, `lib()` raises
and nothing of the engine runs.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_longlong, c_void_p

from .build import ensure_built

P = c_void_p
I = c_int
L = c_longlong
F = c_float
STREAM = c_void_p

_SIGNATURES = {
    "fb_last_error": (c_char_p, []),
    "fb_abi_version": (I, []),
    "fb_copy_rows_to_device": (I, [P, L, P, L, L, L, STREAM]),
    "fb_set_pdl": (None, [I]),
    "fb_set_plain_launch_classes": (None, [I]),
    "fb_set_attention_tc": (None, [I]),
    "fb_set_gemm_pair": (None, [I]),
    # elementwise.cu
    "fb_embedding": (I, [P, I, P, P, I, I, I, P, STREAM]),
    "fb_add_rmsnorm": (I, [P, P, I, I, L, P, I, P, I, P, I, I, F, F, STREAM]),
    "fb_rope_table": (I, [P, P, P, P, I, I, STREAM]),
    "fb_rope_kv_write": (I, [P, L, I, L, P, L, P, L, P, L, I, I, P, P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, P, STREAM]),
    "fb_gate_mul": (I, [P, L, I, I, L, P, I, I, I, I, STREAM]),
    # gemm_simt.cu
    "fb_gemm_simt": (I, [P, I, L, P, I, L, P, I, L, I, I, I, STREAM]),
    # gemm_tc.cu
    "fb_gemm_tc_add": (I, [P, L, P, L, P, L, I, I, I, I, P, STREAM]),
    "fb_gemm_tc": (I, [P, L, P, L, P, I, L, L, I, P, I, I, I, P, L, P, I, I, P, STREAM]),
    "fb_gemm_tc_gated": (I, [P, L, P, L, P, I, L, I, I, I, I, P, L, P, I, P, STREAM]),
    # attention_simt.cu
    "fb_paged_attention_simt": (I, [P, L, P, L, I, P, P, I, I, P, I, P, P, P, I, I, I, I, I, F, P, P, STREAM]),
    # attention_mma.cu
    "fb_paged_attention_mma": (I, [P, L, P, L, P, P, I, I, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P, P, L, P, L,
                                   L, I, P, STREAM]),
    # sampling.cu
    "fb_apply_penalties": (I, [P, L, I, P, P, P, P, P, P, I, STREAM]),
    "fb_apply_logit_bias": (I, [P, L, I, P, P, P, I, STREAM]),
    "fb_sample": (I, [P, L, I, I, P, P, P, P, P, P, STREAM]),
    # host side of the cache manager and of a step's descriptor (csrc/host_cache.cpp)
    "fbh_last_error": (c_char_p, []),
    "fbh_cache_new": (P, [I, P, P, I, I, I]),
    "fbh_cache_free": (None, [P]),
    "fbh_has_slot": (I, [P]),
    "fbh_admit": (I, [P]),
    "fbh_admit_at": (I, [P, I, P]),
    "fbh_release": (I, [P, I]),
    "fbh_length": (I, [P, I]),
    "fbh_reserved_to": (I, [P, I]),
    "fbh_free_pages": (I, [P, P]),
    "fbh_pool_pages": (I, [P, I]),
    "fbh_is_held": (I, [P, I, I]),
    "fbh_pages_needed": (I, [P, I, I, P]),
    "fbh_reserve_all": (I, [P, I, P, P, I]),
    "fbh_commit": (I, [P, I, P, P]),
    "fbh_pages": (I, [P, I, I, P, I]),
    "fbh_first_live_page": (I, [P, I, I]),
    "fbh_check_invariants": (I, [P]),
    "fbh_build_step": (I, [P, I, P, P, P, P, P, I, I, I, I, P, P, P, P, P]),
}

_LIB = None


class KernelError(RuntimeError):
    pass


def declare(handle, signatures: dict) -> None:
    for name, (res, args) in signatures.items():
        try:
            fn = getattr(handle, name)
        except AttributeError:
            raise KernelError(f"the kernel library has no symbol '{name}' (stale build?)") from None
        fn.restype = res
        fn.argtypes = args


def lib():
    """The loaded library (built on first use)."""
    global _LIB
    if _LIB is None:
        path = ensure_built()
        try:
            handle = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        declare(handle, _SIGNATURES)
        if os.environ.get("FLAMBEAU_PDL", "1") == "0":
            handle.fb_set_pdl(0)                # plain stream-ordered launches (for debugging and A/B timing)
        if os.environ.get("FLAMBEAU_PDL_PLAIN"):
            # bit set of kernel classes launched plainly: 1 two-SM product, 2 tcgen05 attention, 4 256-token one-SM product
            handle.fb_set_plain_launch_classes(int(os.environ["FLAMBEAU_PDL_PLAIN"]))
        _LIB = handle
    return _LIB


def library_path() -> str:
    return str(ensure_built())


LAUNCHES = [0]          # launcher calls that reached the device queue (each is at least one kernel launch)

# A section timer (measure.timers.SectionTimer) sets this to be told of every launcher call, after the call has
# queued its kernels: on_launch(what, note), `note` being what the wrapper knows of the call's shape.
ON_LAUNCH = [None]


def check(code: int, what: str, note=None) -> None:
    LAUNCHES[0] += 1
    if code != 0:
        msg = lib().fb_last_error().decode(errors="replace")
        raise KernelError(f"{what}: {msg or 'error code %d' % code}")
    if ON_LAUNCH[0] is not None:
        ON_LAUNCH[0](what, note)
