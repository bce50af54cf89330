"""numpy front-end of the CPU oracle (TEST INFRASTRUCTURE — never the product).

Only the tests, ``__graft_entry__.smoke()`` and the benchmark's CPU-baseline leg
may import this module. It loads ``oracle/_build/libqkan_oracle.so`` (built by
``oracle/build_oracle.py`` from ``qkan_oracle.c``) through ctypes.

The arithmetic restated is the reference's ``pz_encoding`` circuit
(``src/qkan/solver/exact.py:90-134``) followed by the layer epilogue
(``src/qkan/qkan.py:750-785``); see the header of ``qkan_oracle.c`` for the
line-by-line map. Parity pin: reference outputs stored under ``tests/golden/``
(the reference ships no golden vectors of its own for this path).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

from . import build_oracle

PREACT_TRAINABLE = 1
FAST_MEASURE = 2
USE_POSTACT_BIAS = 4

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build_oracle.build())
    return _lib


def num_threads() -> int:
    return int(lib().qkan_oracle_num_threads_f32())


def use_all_cores() -> int:
    """Run the OpenMP loops on every core this process may use (overrides OMP_NUM_THREADS=1 set by launchers)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover
        n = os.cpu_count() or 1
    lib().qkan_oracle_set_num_threads_f32(n)
    return num_threads()


ANSATZ_CODES = {"pz_encoding": 0, "pz": 0, "rpz_encoding": 1, "rpz": 1, "real": 2}


def _flags(preact_trainable: bool, fast_measure: bool, use_postact_bias: bool, ansatz: str = "pz") -> int:
    return ((PREACT_TRAINABLE if preact_trainable else 0) | (FAST_MEASURE if fast_measure else 0)
            | (USE_POSTACT_BIAS if use_postact_bias else 0) | (ANSATZ_CODES[ansatz] << 8))


def _reps_of(theta: np.ndarray, ansatz: str) -> int:
    """Repetitions from the theta shape: (O,I,R+1,2) pz, (O,I,R+1,1) rpz, (O,I,R,1) real."""
    code = ANSATZ_CODES[ansatz]
    if theta.ndim != 4 or theta.shape[3] != (2 if code == 0 else 1):
        raise ValueError(f"theta shape {theta.shape} does not fit ansatz {ansatz!r}")
    return theta.shape[2] - (0 if code == 2 else 1)


def _prep(a, dt):
    if a is None:
        return None, None
    arr = np.ascontiguousarray(np.asarray(a), dtype=dt)
    return arr, arr.ctypes.data_as(ctypes.c_void_p)


def _suffix(dtype) -> str:
    dtype = np.dtype(dtype)
    if dtype == np.float64:
        return "f64"
    if dtype == np.float32:
        return "f32"
    raise ValueError(f"oracle computes in float32 or float64, not {dtype}")


def postacts(x, theta, pw, pb, *, preact_trainable: bool, fast_measure: bool = True,
             dtype=np.float64, ansatz: str = "pz") -> np.ndarray:
    """Per-edge activations ``(B, O, I)`` — the reference solver contract (solver/_base.py:29-51)."""
    sfx = _suffix(dtype)
    x_, xp = _prep(x, dtype)
    th_, thp = _prep(theta, dtype)
    pw_, pwp = _prep(pw, dtype)
    pb_, pbp = _prep(pb, dtype)
    B, I = x_.shape
    O, I2 = th_.shape[:2]
    assert I2 == I
    R = _reps_of(th_, ansatz)
    out = np.empty((B, O, I), dtype=dtype)
    rc = getattr(lib(), f"qkan_oracle_postacts_{sfx}")(
        B, I, O, R, _flags(preact_trainable, fast_measure, False, ansatz), xp, thp, pwp, pbp,
        out.ctypes.data_as(ctypes.c_void_p))
    if rc != 0:
        raise RuntimeError(f"oracle postacts failed ({rc})")
    return out


def forward(x, theta, pw, pb, postw, postb=None, basew=None, mask=None, *, preact_trainable: bool,
            fast_measure: bool = True, use_postact_bias: bool = False, dtype=np.float64,
            ansatz: str = "pz") -> np.ndarray:
    """Layer output ``y (B, O)`` (qkan.py:750-785)."""
    sfx = _suffix(dtype)
    x_, xp = _prep(x, dtype)
    th_, thp = _prep(theta, dtype)
    pw_, pwp = _prep(pw, dtype)
    pb_, pbp = _prep(pb, dtype)
    w_, wp = _prep(postw, dtype)
    b_, bp = _prep(postb, dtype)
    bw_, bwp = _prep(basew, dtype)
    m_, mp = _prep(mask, dtype)
    B, I = x_.shape
    O = th_.shape[0]
    R = _reps_of(th_, ansatz)
    y = np.empty((B, O), dtype=dtype)
    rc = getattr(lib(), f"qkan_oracle_forward_{sfx}")(
        B, I, O, R, _flags(preact_trainable, fast_measure, use_postact_bias, ansatz), xp, thp, pwp, pbp, wp,
        bp, bwp, mp, y.ctypes.data_as(ctypes.c_void_p))
    if rc != 0:
        raise RuntimeError(f"oracle forward failed ({rc})")
    return y


def backward(x, theta, pw, pb, postw, postb, basew, mask, gy, *, preact_trainable: bool,
             fast_measure: bool = True, use_postact_bias: bool = False, dtype=np.float64,
             gpostacts: Optional[np.ndarray] = None, ansatz: str = "pz") -> dict:
    """All gradients of ``sum(y * gy)``; with ``gpostacts`` the cotangent of the ``(B,O,I)`` tensor instead.

    Returns a dict with keys x, theta, preacts_weight, preacts_bias, postact_weights,
    postact_bias, base_weight (the last three are zero when ``gpostacts`` is given).
    """
    sfx = _suffix(dtype)
    x_, xp = _prep(x, dtype)
    th_, thp = _prep(theta, dtype)
    pw_, pwp = _prep(pw, dtype)
    pb_, pbp = _prep(pb, dtype)
    w_, wp = _prep(postw, dtype)
    b_, bp = _prep(postb, dtype)
    bw_, bwp = _prep(basew, dtype)
    m_, mp = _prep(mask, dtype)
    gy_, gyp = _prep(gy, dtype)
    gpa_, gpap = _prep(gpostacts, dtype)
    B, I = x_.shape
    O = th_.shape[0]
    R = _reps_of(th_, ansatz)
    out = {
        "x": np.zeros((B, I), dtype),
        "theta": np.zeros(th_.shape, dtype),
        "preacts_weight": np.zeros((O, I, R), dtype),
        "preacts_bias": np.zeros((O, I, R), dtype),
        "postact_weights": np.zeros((O, I), dtype),
        "postact_bias": np.zeros((O, I), dtype),
        "base_weight": np.zeros((O, I), dtype),
    }
    ptr = {k: v.ctypes.data_as(ctypes.c_void_p) for k, v in out.items()}
    rc = getattr(lib(), f"qkan_oracle_backward_{sfx}")(
        B, I, O, R, _flags(preact_trainable, fast_measure, use_postact_bias, ansatz), xp, thp, pwp, pbp, wp,
        bp, bwp, mp, gyp, gpap, ptr["x"], ptr["theta"], ptr["preacts_weight"], ptr["preacts_bias"],
        ptr["postact_weights"], ptr["postact_bias"], ptr["base_weight"])
    if rc != 0:
        raise RuntimeError(f"oracle backward failed ({rc})")
    return out
