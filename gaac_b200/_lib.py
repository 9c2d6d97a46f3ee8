"""ctypes binding of libgaac_b200.so (the C ABI declared in include/gaac_b200.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""
from __future__ import annotations
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("GAAC_B200_LIB") or os.path.join(_HERE, "libgaac_b200.so")     # GAAC_B200_LIB: use a library built elsewhere
_lib = None

vp, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t


class Side(C.Structure):
    """gaac_side"""
    _fields_ = [("sm", vp), ("codes", vp), ("flags", vp), ("tile_off", vp), ("ovf", vp), ("head_start", vp),
                ("ovf_bytes", i64), ("base3", vp), ("base4", vp), ("tail", vp)]


class Store(C.Structure):
    """gaac_store"""
    _fields_ = [("sm", vp), ("codes", vp), ("flags", vp), ("tile_off", vp), ("ovf", vp), ("ovf_used", vp), ("tail", vp),
                ("base3", vp), ("base4", vp)]


class Paged(C.Structure):
    """gaac_paged"""
    _fields_ = [("buf", vp), ("raw", vp), ("mt", vp), ("stack", vp), ("top", vp), ("err", vp),
                ("b3k", vp), ("b4k", vp), ("b3v", vp), ("b4v", vp), ("n_kv", i32), ("TS", i32), ("ovf_slot", i32)]


class Exchange(C.Structure):
    """gaac_exchange"""
    _fields_ = [("recv", vp), ("epoch", vp), ("ticket", vp), ("err", vp), ("rank", i32), ("world", i32), ("rows_cap", i32)]


_SIGNATURES = {
    "gaac_status_string": (C.c_char_p, [i32]),
    "gaac_abi_version": (i32, []),
    "gaac_encode_tiles": (i32, [vp, i64, i64, i64, i64, vp, vp, vp, i32, i32, vp, vp, vp, vp, vp, vp]),
    "gaac_compact": (i32, [vp, vp, i64, i64, vp, vp, vp, i64, vp, vp, i64, i64, vp, vp]),
    "gaac_head_prefix": (i32, [vp, i64, vp, vp]),
    "gaac_encode_begin": (i32, [vp, i64, i64, i64, i64, vp, vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
    "gaac_compact_copy": (i32, [vp, vp, i64, i64, vp, vp, vp, i64, vp, i64, i64, vp, i32, i64, i64, vp, vp]),
    "gaac_decode_page": (i32, [vp, vp, vp, vp, i64, vp, vp, vp, vp, vp, i32, i32, i64, i64, i64, vp, vp]),
    "gaac_exponent_hist": (i32, [vp, i64, i64, vp, vp]),
    "gaac_bases_from_hist": (i32, [vp, i64, vp, vp, vp]),
    "gaac_set_launch_overlap": (None, [i32]),
    "gaac_attn_workspace_bytes": (sz, [i32, i32, i32]),
    "gaac_attn_workspace_header_bytes": (sz, [i32, i32]),
    "gaac_decode_attn_pages": (i32, [C.POINTER(Side), C.POINTER(Side), vp, i32, i32, i32, i64, i64, f32, i32, i32, vp, sz, vp, vp, vp, C.POINTER(Exchange), i32, vp]),
    "gaac_decode_attn_exchange": (i32, [C.POINTER(Side), C.POINTER(Side), vp, vp, i32, i32, i32, vp, i64, f32, i32, vp, i32, i32, vp, sz, C.POINTER(Exchange), vp, vp, vp]),
    "gaac_debug_decode_attn_rebuild": (i32, [C.POINTER(Side), C.POINTER(Side), vp, vp, i32, i32, i32, vp, i64, i64, f32, i32, vp, i32, i32, vp, sz, vp, vp, vp, vp, i64, vp]),
    "gaac_debug_paged_decode_attn_rebuild": (i32, [C.POINTER(Paged), vp, i64, vp, vp, i32, i32, f32, i32, vp, sz, vp, vp, vp, vp, i64, vp]),
    "gaac_decode_attn": (i32, [C.POINTER(Side), C.POINTER(Side), vp, vp, i32, i32, i32, vp, i64, f32, i32, vp, i32, i32, vp, sz, vp, vp, vp]),
    "gaac_decode_attn_partial": (i32, [C.POINTER(Side), C.POINTER(Side), vp, vp, i32, i32, i32, vp, i64, f32, i32, vp, i32, i32, vp, sz, vp, vp]),
    "gaac_combine": (i32, [vp, vp, vp, i64, i32, vp, vp, vp]),
    "gaac_combine_parts": (i32, [vp, i64, i32, vp, vp, vp]),
    "gaac_decode_attn_push": (i32, [C.POINTER(Side), C.POINTER(Side), vp, vp, i32, i32, i32, vp, i64, f32, i32, vp, i32, i32, vp, sz, C.POINTER(Exchange), vp]),
    "gaac_exchange_merge": (i32, [C.POINTER(Exchange), i64, vp, vp, vp]),
    "gaac_append_kv": (i32, [C.POINTER(Store), C.POINTER(Store), vp, vp, vp, i32, i32, vp, vp, i64, i64, i32, vp, vp]),
    "gaac_cache_prefill_scratch_bytes": (C.c_size_t, [i64, i32]),
    "gaac_cache_prefill": (i32, [C.POINTER(Store), C.POINTER(Store), vp, vp, i64, i64, i32, i32, vp, vp, i64, i64, i32, vp, C.c_size_t, vp, i32, vp]),
    "gaac_paged_store": (i32, [C.POINTER(Paged), vp, vp, i64, i64, vp, i32, vp, vp]),
    "gaac_paged_release": (i32, [C.POINTER(Paged), vp, i32, vp]),
    "gaac_paged_decode_blocks": (i32, [C.POINTER(Paged), vp, i32, vp, vp, i64, vp]),
    "gaac_paged_decode_attn": (i32, [C.POINTER(Paged), vp, i64, vp, vp, i32, i32, f32, i32, vp, sz, vp, vp, vp]),
    "gaac_paged_decode_attn256": (i32, [C.POINTER(Paged), vp, i64, vp, vp, i32, i32, f32, i32, vp, sz, vp, vp, vp]),
    "gaac_decode_attn_static": (i32, [C.POINTER(Side), C.POINTER(Side), vp, vp, i32, i32, i32, vp, i64, f32, i32, vp, i32, i32, vp, vp, vp]),
    "gaac_static_workspace_bytes": (sz, []),
    "gaac_static_workspace_error": (i32, [vp, i32, vp]),
}
EXPORTS = tuple(_SIGNATURES)
ABI_VERSION = 4


def lib():
    """The loaded library.  Raises RuntimeError when it has not been built (python -m gaac_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m gaac_b200.build` (needs nvcc); there is no fallback path")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        if L.gaac_abi_version() != ABI_VERSION:
            raise RuntimeError(f"{LIB_PATH} has ABI version {L.gaac_abi_version()}, this package binds version {ABI_VERSION}: rebuild it (python -m gaac_b200.build --force)")
        _lib = L
    return _lib


def check(status: int, what: str):
    if status != 0:
        raise RuntimeError(f"{what}: {lib().gaac_status_string(status).decode()} (status {status})")


def row_stride(t) -> int:
    """Stride of dim 0 in elements as the library wants it.  torch is free to report anything for a dimension of size 1 (a
    one-row tensor often comes back with the stride of its second dimension), and the library checks the stride against the row
    width: a tensor with at most one row gets the width of a packed row instead."""
    if t.shape[0] > 1:
        return t.stride(0)
    n = 1
    for s in t.shape[1:]:
        n *= s
    return max(n, 1)


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr(device=None):
    import torch
    return torch.cuda.current_stream(device).cuda_stream
