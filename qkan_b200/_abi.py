"""ctypes binding of ``libqkan_b200.so`` (the C ABI in ``include/qkan_b200.h``).

The library is the only compute path of this package: if it cannot be loaded the
import of a compute entry point raises, there is no eager or CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import Structure, c_char_p, c_int, c_int32, c_size_t, c_uint32, c_void_p

QK_ABI_VERSION = 4

QK_F32 = 0
QK_BF16 = 1

QK_ANSATZ_PZ = 0
QK_ANSATZ_RPZ = 1
QK_ANSATZ_REAL = 2
ANSATZ_CODES = {"pz_encoding": QK_ANSATZ_PZ, "pz": QK_ANSATZ_PZ, "rpz_encoding": QK_ANSATZ_RPZ,
                "rpz": QK_ANSATZ_RPZ, "real": QK_ANSATZ_REAL}

QK_PREACT_TRAINABLE = 1
QK_FAST_MEASURE = 2
QK_USE_POSTACT_BIAS = 4
QK_PRECISE_MATH = 8
QK_SINGLE_TABLE = 16

(QK_DBG_BWD_GROUPS, QK_DBG_BWD_RPG, QK_DBG_BWD_RU, QK_DBG_BWD_OSPLIT, QK_DBG_NO_XTRIG, QK_DBG_VERBOSE,
 QK_DBG_FWD_THREADS, QK_DBG_FWD_TB, QK_DBG_FWD_OT, QK_DBG_FWD_ICH) = range(10)

QK_OK = 0
QK_ERR_BAD_ARGUMENT = -1
QK_ERR_UNSUPPORTED = -2
QK_ERR_WORKSPACE = -3
QK_ERR_LAUNCH = -4

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libqkan_b200.so")

# Every symbol include/qkan_b200.h declares, with its C signature.
_P = c_void_p
SYMBOLS = {
    "qk_abi_version": (c_int, []),
    "qk_last_error": (c_char_p, []),
    "qk_forward_workspace_bytes": (c_size_t, [_P]),
    "qk_backward_workspace_bytes": (c_size_t, [_P]),
    "qk_pz_forward": (c_int, [_P] * 10 + [_P, c_size_t, _P]),
    "qk_pz_backward": (c_int, [_P] * 17 + [_P, c_size_t, _P]),
    "qk_pz_postacts_forward": (c_int, [_P] * 6 + [_P, c_size_t, _P]),
    "qk_pz_postacts_backward": (c_int, [_P] * 10 + [_P, c_size_t, _P]),
    "qk_tables_bytes": (c_size_t, [_P]),
    "qk_backward_scratch_bytes": (c_size_t, [_P]),
    "qk_pz_prepare": (c_int, [_P] * 8 + [_P, c_size_t, _P]),
    "qk_pz_forward_prepared": (c_int, [_P, _P, _P, c_size_t, c_int, _P, _P]),
    "qk_pz_backward_prepared": (c_int, [_P, _P, _P, c_size_t, _P, _P, _P, c_int] + [_P] * 8 + [_P, c_size_t, _P]),
    "qk_edge_stats_scratch_bytes": (c_size_t, [_P]),
    "qk_pz_edge_stats": (c_int, [_P, _P, _P, c_size_t, c_int, _P, _P, c_size_t, _P]),
    "qk_debug_set": (None, [c_int, c_int]),
    "qk_noalloc_max_scratch_bytes": (c_size_t, []),
    "qk_noalloc_last_error": (c_char_p, []),
    "qk_pz_forward_noalloc": (c_int, [_P] * 10 + [_P]),
}


class QkDesc(Structure):
    _fields_ = [
        ("batch", c_int32),
        ("in_dim", c_int32),
        ("out_dim", c_int32),
        ("reps", c_int32),
        ("io_dtype", c_int32),
        ("param_dtype", c_int32),
        ("flags", c_uint32),
        ("ansatz", c_int32),
        ("group", c_int32),
    ]


class QkanLibraryError(RuntimeError):
    """The CUDA library is missing, has the wrong ABI, or a call into it failed."""


_lib = None


def load() -> ctypes.CDLL:
    """Load the library once; raise ``QkanLibraryError`` when it is absent or mismatched."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise QkanLibraryError(
            f"{LIB_PATH} not found: build it with `python -m qkan_b200.build` "
            "(this package has no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SYMBOLS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise QkanLibraryError(f"{LIB_PATH} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.qk_abi_version() != QK_ABI_VERSION:
        raise QkanLibraryError(
            f"ABI mismatch: library {lib.qk_abi_version()}, binding {QK_ABI_VERSION}; rebuild")
    _lib = lib
    return lib


def last_error() -> str:
    return load().qk_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc == QK_OK:
        return
    msg = f"{what} failed ({rc}): {last_error()}"
    if rc == QK_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    if rc == QK_ERR_BAD_ARGUMENT:
        raise ValueError(msg)
    raise QkanLibraryError(msg)


def desc_pointer(desc: QkDesc):
    return ctypes.cast(ctypes.pointer(desc), c_void_p)


__all__ = [name for name in dir() if name.startswith("QK") or name in (
    "QkDesc", "QkanLibraryError", "ANSATZ_CODES", "load", "last_error", "check", "desc_pointer", "SYMBOLS", "LIB_PATH")]
