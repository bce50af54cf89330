"""Helpers shared by the tests: golden-case loading, seeded inputs, the error metric."""
from __future__ import annotations

import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

GRAD_NAMES = ("x", "theta", "preacts_weight", "preacts_bias", "postact_weights", "postact_bias",
              "base_weight")

# normalised max error bounds: max|a-b| / max|b|
TOL_F32 = 1e-5
TOL_BF16 = 2e-2


def nerr(a, b) -> float:
    """max|a-b| / max|b| (the per-tensor metric of the parity protocol); absolute when b == 0."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.size == 0:
        return 0.0
    den = np.abs(b).max()
    num = np.abs(a - b).max()
    return float(num if den == 0 else num / den)


def golden_layer_cases():
    d = np.load(os.path.join(GOLDEN, "layer_cases.npz"))
    cases = []
    for name in d["names"]:
        name = str(name)
        g = {k.split("/", 1)[1]: d[k] for k in d.files if k.startswith(name + "/")}
        ptr, fast, use_pb, base, masked = (bool(v) for v in g["flags"])
        g["cfg"] = dict(preact_trainable=ptr, fast_measure=fast, use_postact_bias=use_pb)
        g["base"] = base
        g["masked"] = masked
        g["name"] = name
        cases.append(g)
    return cases


def case_inputs(g):
    """Positional oracle/kernel inputs of a golden case (None where the reference skips the term)."""
    return dict(
        x=g["in_x"], theta=g["in_theta"], pw=g["in_preacts_weight"], pb=g["in_preacts_bias"],
        postw=g["in_postact_weights"],
        postb=g["in_postact_bias"] if g["cfg"]["use_postact_bias"] else None,
        basew=g["in_base_weight"] if g["base"] else None,
        mask=g["in_mask"] if g["masked"] else None,
        gy=g["in_gy"],
    )


def random_problem(seed, B, I, O, R, *, use_pb=True, base=False, masked=False, x_scale=1.0):
    """Seeded inputs with the value distributions of the layer microbenchmark."""
    rng = np.random.default_rng(seed)
    p = dict(
        x=rng.uniform(-x_scale, x_scale, (B, I)),
        theta=rng.uniform(-np.pi, np.pi, (O, I, R + 1, 2)),
        pw=1.0 + 0.2 * rng.standard_normal((O, I, R)),
        pb=0.2 * rng.standard_normal((O, I, R)),
        postw=rng.standard_normal((O, I)) / np.sqrt(max(I, 1)),
        postb=0.3 * rng.standard_normal((O, I)) if use_pb else None,
        basew=0.5 * rng.standard_normal((O, I)) if base else None,
        mask=(rng.uniform(size=(O, I)) > 0.25).astype(np.float64) if masked else None,
        gy=rng.standard_normal((B, O)),
    )
    return {k: (None if v is None else v.astype(np.float32)) for k, v in p.items()}


def golden_ansatz_cases():
    """rpz / real fixtures: inputs, y, postacts and all gradients from the reference (float64)."""
    d = np.load(os.path.join(GOLDEN, "ansatz_cases.npz"))
    cases = []
    for name in d["names"]:
        name = str(name)
        g = {k.split("/", 1)[1]: d[k] for k in d.files if k.startswith(name + "/")}
        ptr, fast = (bool(v) for v in g["flags"])
        g["cfg"] = dict(preact_trainable=ptr, fast_measure=fast, use_postact_bias=True, ansatz=str(g["ansatz"]))
        g["name"] = name
        cases.append(g)
    return cases


def ansatz_case_inputs(g):
    return dict(x=g["in_x"], theta=g["in_theta"], pw=g["in_preacts_weight"], pb=g["in_preacts_bias"],
                postw=g["in_postact_weights"], postb=g["in_postact_bias"], basew=g["in_base_weight"],
                mask=g["in_mask"], gy=g["in_gy"])


def golden_group_cases():
    """Grouped theta / preacts ``(g, ...)`` run through the reference's exact solver (float64 / complex128)."""
    d = np.load(os.path.join(GOLDEN, "group_cases.npz"))
    cases = []
    for name in d["names"]:
        name = str(name)
        g = {k.split("/", 1)[1]: d[k] for k in d.files if k.startswith(name + "/")}
        ptr, fast = (bool(v) for v in g["flags"])
        g["cfg"] = dict(preact_trainable=ptr, fast_measure=fast, use_postact_bias=True, ansatz=str(g["ansatz"]))
        g["name"] = name
        cases.append(g)
    return cases


def expand_group(t, out_dim: int, in_dim: int):
    """(g, ...) -> (O, I, ...) with entry ``i mod g`` on edge (o, i): the broadcast the reference solvers apply."""
    idx = np.arange(in_dim) % t.shape[0]
    return np.broadcast_to(t[idx][None], (out_dim, in_dim) + t.shape[1:]).copy()


def reduce_group(g_edge, group: int):
    """Sum per-edge gradients (O, I, ...) over the edges sharing an entry -> (g, ...)."""
    out = np.zeros((group,) + g_edge.shape[2:], dtype=g_edge.dtype)
    for i in range(g_edge.shape[1]):
        out[i % group] += g_edge[:, i].sum(axis=0)
    return out
