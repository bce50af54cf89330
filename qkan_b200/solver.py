"""The kernels as a solver plug-in in the reference's sense.

The reference dispatches through a string-keyed registry of callables
``solver(x, theta, preacts_weight, preacts_bias, reps, **kwargs) -> (B, O, I)``
(``src/qkan/solver/_base.py:29-70``; call site ``src/qkan/qkan.py:699-714``).
``B200Solver`` implements that contract on the CUDA kernels; a small registry with the
same three functions lives here, and ``register_with_reference()`` adds the solver to
the reference's own registry when that package is installed next to this one.
"""
from __future__ import annotations

import torch

from . import functional as qf

_SUPPORTED = ("pz_encoding", "pz", "rpz_encoding", "rpz", "real")


class B200Solver:
    """``solver="b200"``: per-edge activations (pz, rpz and real ansaetze) on the sm_100a kernels."""

    name = "b200"

    def __call__(self, x, theta, preacts_weight, preacts_bias, reps, **kwargs) -> torch.Tensor:
        ansatz = kwargs.get("ansatz", "pz_encoding")
        if callable(ansatz) or ansatz not in _SUPPORTED:
            raise NotImplementedError(
                f"the b200 solver implements pz_encoding, rpz_encoding and real, got {ansatz!r}")
        trainable = kwargs.get("preacts_trainable", False)
        fast = kwargs.get("fast_measure", True)
        batch, in_dim = x.shape
        out_dim = kwargs.get("out_dim", in_dim)
        layers = reps if ansatz == "real" else reps + 1
        if theta.dim() == 3 and preacts_weight.dim() == 2 and theta.shape[0] == preacts_weight.shape[0]:
            # grouped parameters (g, ...): the kernels index entry i mod g themselves and reduce the
            # gradients per entry, so nothing of size (O, I, ...) is materialised
            if theta.shape[1] != layers:
                raise ValueError(f"theta holds {theta.shape[1]} layers, reps={reps} needs {layers}")
            return qf.qkan_postacts(x, theta, preacts_weight, preacts_bias, preact_trainable=trainable,
                                    fast_measure=fast, ansatz=ansatz, precise=kwargs.get("precise", "auto"),
                                    out_dim=out_dim)
        # mixed shapes: broadcast as the reference solvers do (src/qkan/solver/exact.py:68-86)
        if theta.dim() != 4:
            theta = theta.unsqueeze(0)
        if theta.shape[1] != in_dim or theta.shape[0] != out_dim:
            rep_in = in_dim // theta.shape[1] + 1
            rep_out = out_dim if theta.shape[0] == 1 else 1
            theta = theta.repeat(rep_out, rep_in, 1, 1)[:, :in_dim]
        if preacts_weight.dim() != 3:
            preacts_weight, preacts_bias = preacts_weight.unsqueeze(0), preacts_bias.unsqueeze(0)
        if preacts_weight.shape[1] != in_dim or preacts_weight.shape[0] != out_dim:
            rep_in = in_dim // preacts_weight.shape[1] + 1
            rep_out = out_dim if preacts_weight.shape[0] == 1 else 1
            preacts_weight = preacts_weight.repeat(rep_out, rep_in, 1)[:, :in_dim]
            preacts_bias = preacts_bias.repeat(rep_out, rep_in, 1)[:, :in_dim]
        if theta.shape[2] != layers:
            raise ValueError(f"theta holds {theta.shape[2]} layers, reps={reps} needs {layers}")
        return qf.qkan_postacts(x, theta, preacts_weight, preacts_bias, preact_trainable=trainable,
                                fast_measure=fast, ansatz=ansatz, precise=kwargs.get("precise", "auto"))


_REGISTRY: dict = {}


def register(solver):
    """Register a solver instance under its ``name`` (``src/qkan/solver/_base.py:57-60``)."""
    _REGISTRY[solver.name] = solver
    return solver


def get_solver(name: str):
    return _REGISTRY[name]


def get_registry() -> dict:
    return _REGISTRY


register(B200Solver())


def register_with_reference() -> bool:
    """Add the solver to the reference package's registry; False when that package is absent."""
    try:
        from qkan.solver import register as ref_register  # type: ignore
    except Exception:
        return False
    ref_register(get_solver("b200"))
    return True
