"""The CPU oracle against the reference's own outputs (tests/golden, made by make_golden.py)."""
import numpy as np
import pytest

from oracle import oracle
from tests.util import (GRAD_NAMES, ansatz_case_inputs, case_inputs, expand_group, golden_ansatz_cases,
                        golden_group_cases, golden_layer_cases, nerr, reduce_group)


@pytest.mark.parametrize("case", golden_layer_cases(), ids=lambda c: c["name"])
def test_oracle_f64_matches_reference(case):
    p = case_inputs(case)
    args = [p[k] for k in ("x", "theta", "pw", "pb", "postw", "postb", "basew", "mask")]
    y = oracle.forward(*args, **case["cfg"])
    assert nerr(y, case["y"]) <= 1e-13
    pa = oracle.postacts(p["x"], p["theta"], p["pw"], p["pb"],
                         preact_trainable=case["cfg"]["preact_trainable"],
                         fast_measure=case["cfg"]["fast_measure"])
    assert nerr(pa, case["postacts"]) <= 1e-13
    g = oracle.backward(*args, p["gy"], **case["cfg"])
    for k in GRAD_NAMES:
        assert nerr(g[k], case["g_" + k]) <= 1e-12, k


@pytest.mark.parametrize("case", golden_layer_cases(), ids=lambda c: c["name"])
def test_oracle_f32_matches_reference_complex64(case):
    """float32 build vs the reference's default complex64 arithmetic."""
    p = case_inputs(case)
    args = [p[k] for k in ("x", "theta", "pw", "pb", "postw", "postb", "basew", "mask")]
    y = oracle.forward(*args, dtype=np.float32, **case["cfg"])
    assert nerr(y, case["y_f32"]) <= 2e-6


def test_oracle_gradients_match_finite_differences():
    rng = np.random.default_rng(0)
    B, I, O, R = 3, 2, 2, 2
    x = rng.uniform(-1, 1, (B, I)); th = rng.uniform(-3, 3, (O, I, R + 1, 2))
    pw = 1 + 0.2 * rng.standard_normal((O, I, R)); pb = 0.2 * rng.standard_normal((O, I, R))
    w = rng.standard_normal((O, I)); b = rng.standard_normal((O, I)); bw = rng.standard_normal((O, I))
    gy = rng.standard_normal((B, O))
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    g = oracle.backward(x, th, pw, pb, w, b, bw, None, gy, **cfg)
    loss = lambda **kw: float((oracle.forward(kw.get("x", x), kw.get("th", th), kw.get("pw", pw), kw.get("pb", pb),  # noqa: E731
                                              w, b, bw, None, **cfg) * gy).sum())
    eps = 1e-6
    for name, arr, key in (("x", x, "x"), ("th", th, "theta"), ("pw", pw, "preacts_weight"), ("pb", pb, "preacts_bias")):
        idx = tuple(0 for _ in arr.shape)
        hi, lo = arr.copy(), arr.copy()
        hi[idx] += eps; lo[idx] -= eps
        fd = (loss(**{name: hi}) - loss(**{name: lo})) / (2 * eps)
        assert abs(fd - g[key][idx]) <= 1e-6 * max(1, abs(fd)), name


def test_oracle_rejects_too_many_reps():
    with pytest.raises(RuntimeError):
        oracle.postacts(np.zeros((1, 1)), np.zeros((1, 1, 66, 2)), np.zeros((1, 1, 65)), np.zeros((1, 1, 65)),
                        preact_trainable=True)


@pytest.mark.parametrize("case", golden_ansatz_cases(), ids=lambda c: c["name"])
def test_oracle_matches_reference_for_rpz_and_real(case):
    p = ansatz_case_inputs(case)
    args = [p[k] for k in ("x", "theta", "pw", "pb", "postw", "postb", "basew", "mask")]
    cfg = case["cfg"]
    assert nerr(oracle.forward(*args, **cfg), case["y"]) <= 1e-13
    pa = oracle.postacts(*args[:4], preact_trainable=cfg["preact_trainable"], fast_measure=cfg["fast_measure"],
                         ansatz=cfg["ansatz"])
    assert nerr(pa, case["postacts"]) <= 1e-13
    g = oracle.backward(*args, p["gy"], **cfg)
    for k in GRAD_NAMES:
        assert nerr(g[k], case["g_" + k]) <= 1e-12, k


@pytest.mark.parametrize("case", golden_group_cases(), ids=lambda c: c["name"])
def test_oracle_with_group_broadcast_matches_reference(case):
    """Pins the grouping rule (entry i mod g for every output) on the reference's own broadcast."""
    cfg = case["cfg"]
    O, I = case["in_postact_weights"].shape
    G = case["in_theta"].shape[0]
    theta, pw, pb = (expand_group(case[k], O, I) for k in ("in_theta", "in_preacts_weight", "in_preacts_bias"))
    args = [case["in_x"], theta, pw, pb, case["in_postact_weights"], case["in_postact_bias"], None, None]
    assert nerr(oracle.forward(*args, **cfg), case["y"]) <= 1e-13
    g = oracle.backward(*args, case["in_gy"], **cfg)
    for k in ("x", "postact_weights", "postact_bias"):
        assert nerr(g[k], case["g_" + k]) <= 1e-12, k
    for k in ("theta", "preacts_weight", "preacts_bias"):
        assert nerr(reduce_group(g[k], G), case["g_" + k]) <= 1e-12, k
