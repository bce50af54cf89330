"""The hybrid block of the HQKANsformer MLP: Linear -> QKAN[w, w] -> Linear.

Mirrors the reference's ``FusedHQKAN`` (``src/qkan/solver/cute/cute_ops.py:449-490``): the same three named
sub-modules (``down``, ``qkan``, ``up``), constructor arguments and defaults, with the QKAN layer on the
``"b200"`` solver. The two projections are plain library GEMMs, as in the reference; the block is bound by
launches at the usual widths, so it is meant to run under ``graph.make_graphed_train_step`` /
``graph.make_graphed_inference``.
"""
from __future__ import annotations

import torch
from torch import nn

from .layer import SOLVER_NAME
from .model import QKAN


class FusedHQKAN(nn.Module):
    """``up(qkan(down(x)))`` with ``down: in_features -> qkan_width`` and ``up`` back again."""

    def __init__(self, in_features: int, qkan_width: int, reps: int = 1, solver: str = SOLVER_NAME,
                 ansatz: str = "pz_encoding", c_dtype: torch.dtype = torch.bfloat16,
                 p_dtype: torch.dtype = torch.bfloat16, device: str = "cuda"):
        super().__init__()
        self.down = nn.Linear(in_features, qkan_width, device=device, dtype=p_dtype)
        self.qkan = QKAN(width=[qkan_width, qkan_width], reps=reps, ba_trainable=True, device=device,
                         solver=solver, ansatz=ansatz, c_dtype=c_dtype, p_dtype=p_dtype)
        self.up = nn.Linear(qkan_width, in_features, device=device, dtype=p_dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.up(self.qkan(self.down(x)))
