"""ctypes binding of libsage3_b200.so (the C ABI declared in include/sage3_b200.h).

The library must have been built (python -m sageattention_b200.build); there is no fallback: if it is
missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import pathlib

_PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = _PKG / "libsage3_b200.so"

SAGE3_FP16, SAGE3_BF16 = 0, 1
ABI_VERSION = 4          # SAGE3_ABI_VERSION of include/sage3_b200.h this module's structs were written for
SAGE3_OK = 0
SAGE3_E_DEVICE_WAIT = -9


class Sage3Desc(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Nq", C.c_int32), ("Nk", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("is_causal", C.c_int32), ("per_block_mean", C.c_int32), ("reserved", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("sm_scale", C.c_float), ("reserved2", C.c_int32), ("sm_scale_per_head", C.c_void_p),
    ]


class Sage3Workspace(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in
                ("status", "kpart", "km", "qm", "delta", "q_codes", "q_sf", "k_codes", "k_sf", "v_codes", "v_sf",
                 "qkm", "total_bytes")] + [(n, C.c_int32) for n in ("nq_pad", "nk_pad", "nqm", "kchunks")]


MAX_PARTS = 8


class Sage3Parts(C.Structure):
    _fields_ = [("parts", C.c_int32), ("rows_per_part", C.c_int32), ("base", C.c_void_p * MAX_PARTS)]


class Sage3Carry(C.Structure):
    _fields_ = [("o_in", C.c_void_p), ("m_in", C.c_void_p), ("l_in", C.c_void_p), ("o_out", C.c_void_p), ("m_out", C.c_void_p),
                ("l_out", C.c_void_p), ("use_causal_shift", C.c_int32), ("causal_shift", C.c_int32)]


class Sage3Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        super().__init__(f"{where}: {lib().sage3_strerror(code).decode()} (code {code})")


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library once.  Raises if it has not been built: there is no CPU or eager path."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing; build it with `python -m sageattention_b200.build` "
            "(needs nvcc with sm_100a support). sageattention_b200 has no fallback path.")
    l = C.CDLL(str(LIB_PATH))
    l.sage3_version.restype = C.c_int
    if l.sage3_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {l.sage3_version()}, this package needs {ABI_VERSION}: rebuild it "
                          "with `python -m sageattention_b200.build`")
    P, V = C.POINTER, C.c_void_p
    l.sage3_version.restype = C.c_int
    l.sage3_version.argtypes = []
    l.sage3_strerror.restype = C.c_char_p
    l.sage3_strerror.argtypes = [C.c_int]
    l.sage3_workspace_layout.restype = C.c_int
    l.sage3_workspace_layout.argtypes = [P(Sage3Desc), P(Sage3Workspace)]
    l.sage3_workspace_bytes.restype = C.c_size_t
    l.sage3_workspace_bytes.argtypes = [P(Sage3Desc)]
    l.sage3_prepass.restype = C.c_int
    l.sage3_prepass.argtypes = [P(Sage3Desc), V, V, V, V, V]
    l.sage3_attn_fwd.restype = C.c_int
    l.sage3_attn_fwd.argtypes = [P(Sage3Desc), V, V, V, V]
    l.sage3_prepass_kmean.restype = C.c_int
    l.sage3_prepass_kmean.argtypes = [P(Sage3Desc), V, V, V, V, V, V]
    l.sage3_prepass_parts.restype = C.c_int
    l.sage3_prepass_parts.argtypes = [P(Sage3Desc), P(Sage3Parts), P(Sage3Parts), P(Sage3Parts), V, V]
    l.sage3_attn_fwd_parts.restype = C.c_int
    l.sage3_attn_fwd_parts.argtypes = [P(Sage3Desc), V, P(Sage3Parts), V, V]
    l.sage3_attn_fwd_carry.restype = C.c_int
    l.sage3_attn_fwd_carry.argtypes = [P(Sage3Desc), V, P(Sage3Carry), V, V, V]
    l.sage3_shared_alloc.restype = C.c_int
    l.sage3_shared_alloc.argtypes = [C.c_size_t, P(C.c_void_p), C.c_char_p]
    l.sage3_shared_open.restype = C.c_int
    l.sage3_shared_open.argtypes = [C.c_char_p, P(C.c_void_p)]
    l.sage3_shared_close.restype = C.c_int
    l.sage3_shared_close.argtypes = [V]
    l.sage3_shared_free.restype = C.c_int
    l.sage3_shared_free.argtypes = [V]
    l.sage3_fwd.restype = C.c_int
    l.sage3_fwd.argtypes = [P(Sage3Desc), V, V, V, V, V, V, V]
    l.sage3_fwd_varlen.restype = C.c_int
    l.sage3_fwd_varlen.argtypes = [P(Sage3Desc), V, V, V, V, V, V, V, V, V]
    l.sage3_mean_from_partial_sums.restype = C.c_int
    l.sage3_mean_from_partial_sums.argtypes = [V, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, V, V]
    l.sage3_selftest_wait_timeout.restype = C.c_int
    l.sage3_selftest_wait_timeout.argtypes = [V, V]
    l.sage3_slab_copy.restype = C.c_int
    l.sage3_slab_copy.argtypes = [V, V, C.c_int32, C.c_int32, C.c_int32, P(C.c_int64 * 3), P(C.c_int64 * 3), C.c_int64, V]
    l.sage3_merge_partial.restype = C.c_int
    l.sage3_merge_partial.argtypes = [V, V, V, V, V, C.c_int64, C.c_int32, C.c_int32, C.c_int32, V]
    l.sage3_kmean_noalloc.restype = C.c_int
    l.sage3_kmean_noalloc.argtypes = [P(Sage3Desc), V, V, V]
    l.sage3_check_status.restype = C.c_int
    l.sage3_check_status.argtypes = [V, P(C.c_int32), V]
    _lib = l
    return l


EXPORTED = ["sage3_version", "sage3_strerror", "sage3_workspace_layout", "sage3_workspace_bytes", "sage3_prepass",
            "sage3_attn_fwd", "sage3_fwd", "sage3_check_status", "sage3_kmean_noalloc", "sage3_selftest_wait_timeout", "sage3_slab_copy", "sage3_merge_partial",
            "sage3_prepass_kmean", "sage3_prepass_parts", "sage3_attn_fwd_parts", "sage3_attn_fwd_carry", "sage3_shared_alloc", "sage3_shared_open",
            "sage3_shared_close", "sage3_shared_free", "sage3_fwd_varlen", "sage3_mean_from_partial_sums"]


def check(code: int, where: str) -> None:
    if code != SAGE3_OK:
        raise Sage3Error(code, where)
