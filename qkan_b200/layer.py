"""``QKANLayer``: the reference's layer interface on top of the fused B200 kernels.

Mirrors ``QKANLayer`` of the reference (``src/qkan/qkan.py:46-957``): same constructor
arguments and defaults (``:106-145``), same parameter names, shapes, ``p_dim`` storage
and seeded initialisation (``:232-386, 475-501``), same ``state_dict`` keys, so a
checkpoint written by either implementation loads into the other. What differs is the
body of ``forward``: the solver call, the mask fold and the epilogue
(``:727-785``) are one CUDA op (``functional.qkan_layer``), selected by
``solver="b200"``. There is no CPU path: calling the layer on a CPU tensor raises.
"""
from __future__ import annotations

import math
import random
import warnings
from typing import Callable, Optional, Union

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from . import functional as qf

SOLVER_NAME = "b200"
_PZ = ("pz_encoding", "pz")
_RPZ = ("rpz_encoding", "rpz")
_SUPPORTED_ANSATZ = _PZ + _RPZ + ("real",)
_ACTIVATIONS = {
    "silu": nn.SiLU, "swish": nn.SiLU,
    "gelu": lambda: nn.GELU(approximate="none"), "gelu_exact": lambda: nn.GELU(approximate="none"),
    "gelu_tanh": lambda: nn.GELU(approximate="tanh"),
    "relu": nn.ReLU, "tanh": nn.Tanh, "sigmoid": nn.Sigmoid,
}


def make_base_activation(kind: str) -> nn.Module:
    """Named base activation (``src/qkan/solver/_activation.py:66-92``); silu is fused in-kernel."""
    try:
        return _ACTIVATIONS[kind.lower()]()
    except KeyError:
        raise ValueError(f"Unknown activation kind {kind!r}. Supported: {sorted(_ACTIVATIONS)}") from None


def _seed_everything(seed) -> None:
    if seed is not None:
        torch.manual_seed(seed)
        np.random.seed(seed)
        random.seed(seed)


class QKANLayer(nn.Module):
    """One QKAN layer ``(B, in_dim) -> (B, out_dim)`` evaluated by the fused sm_100a kernels."""

    _PDIM_RESHAPABLE_NAMES = ("theta", "preacts_weight", "preacts_bias", "base_weight",
                              "postact_weights", "postact_bias", "mask")

    def __init__(self, in_dim: int, out_dim: int, reps: int = 3, group: Union[int, tuple] = -1,
                 device="cpu", solver: Union[str, Callable] = SOLVER_NAME, qml_device="default.qubit",
                 ansatz: Union[str, Callable] = "pz_encoding", theta_size: Optional[list] = None,
                 preact_trainable: bool = False, preact_init: bool = False,
                 postact_weight_trainable: bool = False, postact_bias_trainable: bool = False,
                 base_activation: Union[str, nn.Module] = "silu", ba_trainable: bool = True,
                 is_batchnorm: bool = False, fast_measure: bool = True,
                 c_dtype: torch.dtype = torch.complex64, p_dtype: torch.dtype = torch.float32,
                 seed=None, solver_kwargs: Optional[dict] = None, p_dim: int = 4,
                 checkpoint_reps: bool = False, theta_init: str = "xavier"):
        super().__init__()
        if p_dim not in (2, 4):
            raise ValueError(f"p_dim must be 2 or 4, got {p_dim}")
        if callable(ansatz) or ansatz not in _SUPPORTED_ANSATZ:
            raise NotImplementedError(
                f"ansatz {ansatz!r}: the B200 kernels implement pz_encoding, rpz_encoding and real")
        self.p_dim = p_dim
        self.solver_kwargs = solver_kwargs or {}
        self.checkpoint_reps = checkpoint_reps  # accepted for compatibility; nothing is checkpointed here
        if isinstance(base_activation, str):
            base_activation = make_base_activation(base_activation)
        _seed_everything(seed)
        if isinstance(group, int):
            group = (out_dim, in_dim) if group == -1 else (group,)
        self.in_dim, self.out_dim, self.reps, self.group = in_dim, out_dim, reps, tuple(group)
        self.device = device
        self.solver = solver
        self.qml_device = qml_device
        self.ansatz = ansatz
        self.theta_size = theta_size
        self.base_activation = base_activation
        self.ba_trainable = ba_trainable
        self.is_batchnorm = is_batchnorm
        self.fast_measure = fast_measure
        self.seed = seed
        # c_dtype, the reference's "compute dtype" (src/qkan/qkan.py:203-211, src/qkan/solver/cute/cute_ops.py:191-231):
        #   complex64 / float32 (default)  -> float32 activations in and out of the kernels;
        #   complex128 / float64           -> accepted, computed in float32 (the kernels have no float64 path);
        #   bfloat16                       -> activations cross the kernel boundary as bfloat16 (x, y, their
        #                                     gradients), as in the reference's bf16 mode; theta, preacts and all
        #                                     accumulation stay float32 here (the reference rounds theta to bf16);
        #   float8_e4m3fn                  -> the same as bfloat16: in the reference this value only selects fp8
        #                                     storage of the backward's state checkpoints
        #                                     (src/qkan/csrc/cute_kernels.cu:1283-1292), and this backward keeps no
        #                                     checkpoints at all (it sweeps one torque vector back), so there is
        #                                     nothing left for the value to change.
        known = {torch.complex64: torch.float32, torch.complex128: torch.float64, torch.float32: torch.float32,
                 torch.float64: torch.float64, torch.bfloat16: torch.bfloat16,
                 torch.float8_e4m3fn: torch.float8_e4m3fn}
        if c_dtype not in known:
            raise ValueError(f"c_dtype {c_dtype} is not supported: use complex64 / float32, complex128 / float64, "
                             "bfloat16 or float8_e4m3fn")
        self.c_dtype = known[c_dtype]
        self._io_bf16 = self.c_dtype in (torch.bfloat16, torch.float8_e4m3fn)
        self.p_dtype = p_dtype
        self.preact_trainable = preact_trainable
        self.preact_init = preact_init
        self.postact_weight_trainable = postact_weight_trainable
        self.postact_bias_trainable = postact_bias_trainable
        self.theta_init = theta_init
        self.init_parameters()

    # ------------------------------------------------------------------ parameters
    def init_parameters(self) -> None:
        """Allocate every parameter in the reference's order so that seeded runs match bit for bit."""
        _seed_everything(self.seed)
        group, reps, dev, dt = self.group, self.reps, self.device, self.p_dtype
        self.group_count = int(np.prod(group))
        # theta layers x gates per layer, as in the reference (src/qkan/qkan.py:265-274)
        if self.ansatz in _PZ:
            self._theta_natural_shape = (*group, reps + 1, 2)
        elif self.ansatz in _RPZ:
            self._theta_natural_shape = (*group, reps + 1, 1)
        else:  # "real": no final layer; the reference also pins its compute dtype to bfloat16 here
            self._theta_natural_shape = (*group, reps, 1)
            self.c_dtype = torch.bfloat16  # recorded as the reference does; the activations keep their own dtype here
        self._preacts_natural_shape = (*group, reps)
        flat = self.p_dim == 2
        theta_shape = ((self.group_count, self._theta_natural_shape[-2] * self._theta_natural_shape[-1])
                       if flat else self._theta_natural_shape)
        pre_shape = (self.group_count, reps) if flat else self._preacts_natural_shape
        oi_shape = (self.out_dim * self.in_dim,) if flat else (self.out_dim, self.in_dim)

        self.theta = nn.Parameter(torch.empty(*theta_shape, device=dev, dtype=dt))
        self.preacts_weight = nn.Parameter(torch.ones(*pre_shape, device=dev, dtype=dt),
                                           requires_grad=self.preact_trainable)
        # rpz always trains its encoding bias (src/qkan/qkan.py:292-295)
        self.preacts_bias = nn.Parameter(torch.zeros(*pre_shape, device=dev, dtype=dt),
                                         requires_grad=self.preact_trainable or self.ansatz in _RPZ)
        if self.ba_trainable:
            self.base_weight = nn.Parameter(0.5 * torch.ones(*oi_shape, device=dev, dtype=dt))
        else:
            self.base_weight = nn.Parameter(torch.zeros(*oi_shape, device=dev, dtype=dt), requires_grad=False)
        self.postact_weights = nn.Parameter(torch.ones(*oi_shape, device=dev, dtype=dt),
                                            requires_grad=self.postact_weight_trainable)
        self.postact_bias = nn.Parameter(torch.zeros(*oi_shape, device=dev, dtype=dt),
                                         requires_grad=self.postact_bias_trainable)
        self._pb_is_nonzero = False
        self._bw_is_nonzero = bool(self.ba_trainable)  # a frozen all-zero base weight skips the base term
        self.mask = nn.Parameter(torch.ones(*oi_shape, device=dev, dtype=dt), requires_grad=False)
        self._mask_is_identity = True
        if self.is_batchnorm:
            self.bn = nn.BatchNorm1d(self.in_dim, device=dev, dtype=dt)
        self._x0 = None
        try:
            self.xavier_init()
        except Exception:  # same tolerance as the reference (degenerate fan sizes)
            warnings.warn("xavier_init failed, using default initialization")

    def _theta_natural(self) -> torch.Tensor:
        return self.theta.view(*self._theta_natural_shape) if self.p_dim == 2 else self.theta

    def _preacts_w_natural(self) -> torch.Tensor:
        return self.preacts_weight.view(*self._preacts_natural_shape) if self.p_dim == 2 else self.preacts_weight

    def _preacts_b_natural(self) -> torch.Tensor:
        return self.preacts_bias.view(*self._preacts_natural_shape) if self.p_dim == 2 else self.preacts_bias

    def _as_oi(self, t: torch.Tensor) -> torch.Tensor:
        return t if self.p_dim == 4 else t.view(self.out_dim, self.in_dim)

    def xavier_init(self) -> None:
        if self.theta_init == "small_gaussian":
            nn.init.normal_(self._theta_natural().data, mean=0.0, std=1.0 / math.sqrt(max(self.reps, 1)))
        elif self.theta_init == "xavier":
            nn.init.xavier_normal_(self._theta_natural().data)
        else:
            raise ValueError(f"Unknown theta_init: {self.theta_init!r}")
        if self.preact_init:
            nn.init.xavier_normal_(self._preacts_w_natural().data)
            nn.init.xavier_normal_(self._preacts_b_natural().data)

    def reset_parameters(self) -> None:
        """Reset in place: theta to zero (layer extension), everything else to its default."""
        _seed_everything(self.seed)
        self.theta.data.zero_()
        self.base_weight.data.fill_(0.5 if self.ba_trainable else 0.0)
        self.preacts_weight.data.fill_(1)
        self.preacts_bias.data.zero_()
        self.postact_weights.data.fill_(1)
        self.postact_bias.data.zero_()
        self._pb_is_nonzero = False
        self._bw_is_nonzero = bool(self.ba_trainable)
        self.mask.data.fill_(1)
        self._mask_is_identity = True
        if self.is_batchnorm:
            self.bn.reset_parameters()
        self._x0 = None

    @property
    def param_size(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)

    @property
    def x0(self):
        return self._x0

    @x0.setter
    def x0(self, x):
        self._x0 = None

    # ------------------------------------------------------------------ state dict / device moves
    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        # checkpoints written with the other p_dim hold the same numbers in another shape
        for name in self._PDIM_RESHAPABLE_NAMES:
            key = prefix + name
            target = getattr(self, name, None)
            if key in state_dict and isinstance(target, torch.Tensor):
                src = state_dict[key]
                if src.shape != target.shape and src.numel() == target.numel():
                    state_dict[key] = src.reshape(target.shape)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)
        with torch.no_grad():  # a loaded pruned mask / frozen non-zero bias must not be skipped
            self._mask_is_identity = bool((self.mask == 1).all())
            self._pb_is_nonzero = bool(self.postact_bias.data.any())
            self._bw_is_nonzero = bool(self.ba_trainable or self.base_weight.data.any())

    def to(self, *args, **kwargs):
        for arg in args:
            if isinstance(arg, (str, torch.device)):
                self.device = arg
            elif isinstance(arg, torch.dtype):
                self.p_dtype = arg
        if isinstance(kwargs.get("dtype"), torch.dtype):
            self.p_dtype = kwargs["dtype"]
        if "device" in kwargs:
            self.device = kwargs["device"]
        return super().to(*args, **kwargs)

    def set_fused_epilogue(self, enabled: bool = True) -> None:
        """Kept for interface compatibility: the epilogue is always fused into the kernel here."""

    # ------------------------------------------------------------------ forward
    def _kernel_params(self):
        """theta / preacts as the kernels take them: per edge ``(O, I, ...)``, or grouped ``(g, ...)``.

        A single group axis is passed through as it is: the kernels read entry ``i mod g`` for edge (o, i)
        (the broadcast of ``src/qkan/solver/exact.py:68-86``) and return the gradients already summed per entry.
        """
        theta, pw, pb = self._theta_natural(), self._preacts_w_natural(), self._preacts_b_natural()
        if theta.dim() == 3 and pw.dim() == 2:
            return theta, pw, pb
        return self._expanded()

    def _expanded(self):
        """theta / preacts materialised in the per-edge rank ``(O, I, ...)`` with ``repeat``, exactly as the
        reference solvers do (``src/qkan/solver/exact.py:68-86``); autograd then sums the gradients over the group.
        """
        theta, pw, pb = self._theta_natural(), self._preacts_w_natural(), self._preacts_b_natural()
        if theta.dim() != 4:
            theta = theta.unsqueeze(0)
            pw, pb = pw.unsqueeze(0), pb.unsqueeze(0)
        if theta.shape[1] != self.in_dim or theta.shape[0] != self.out_dim:
            rep_in = self.in_dim // theta.shape[1] + 1
            theta = theta.repeat(self.out_dim, rep_in, 1, 1)[:, : self.in_dim]
            pw = pw.repeat(self.out_dim, rep_in, 1)[:, : self.in_dim]
            pb = pb.repeat(self.out_dim, rep_in, 1)[:, : self.in_dim]
        return theta, pw, pb

    def _check_solver(self) -> None:
        if self.solver != SOLVER_NAME:
            raise NotImplementedError(
                f"solver={self.solver!r}: this package provides the '{SOLVER_NAME}' solver only "
                "(the fused sm_100a kernels); use the reference package for its own solvers")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        assert x.shape[1] == self.in_dim, "Invalid input dimension"
        self._check_solver()
        if self.is_batchnorm:
            x = self.bn(x)
        out_dtype = x.dtype
        if self._io_bf16 and x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)  # c_dtype bfloat16 / float8: bf16 activations at the kernel boundary
        theta, pw, pb = self._kernel_params()
        use_pb = self.postact_bias_trainable or self._pb_is_nonzero
        mask = None if self._mask_is_identity else self._as_oi(self.mask)
        base_w = self._as_oi(self.base_weight)
        has_base = self.ba_trainable or base_w.requires_grad or self._bw_is_nonzero
        silu_base = isinstance(self.base_activation, nn.SiLU)
        y = qf.qkan_layer(
            x, theta, pw, pb, self._as_oi(self.postact_weights),
            self._as_oi(self.postact_bias) if use_pb else None,
            base_w if (has_base and silu_base) else None, mask,
            preact_trainable=self.preact_trainable, fast_measure=self.fast_measure,
            use_postact_bias=use_pb, ansatz=self.ansatz, precise=self.solver_kwargs.get("precise", "auto"))
        if has_base and not silu_base:
            # other base activations stay a plain library GEMM beside the kernel (qkan.py:755, 784)
            w = base_w if mask is None else base_w * mask
            y = y + F.linear(self.base_activation(x), w.to(x.dtype))
        return y if y.dtype == out_dtype else y.to(out_dtype)

    @torch.no_grad()
    def forward_no_sum(self, x: torch.Tensor) -> torch.Tensor:
        """Per-edge outputs ``(B, O, I)`` before the sum over inputs (``src/qkan/qkan.py:835-891``)."""
        assert x.shape[1] == self.in_dim, "Invalid input dimension"
        self._check_solver()
        theta, pw, pb = self._kernel_params()
        postacts = qf.postacts_forward(x, theta, pw, pb, preact_trainable=self.preact_trainable,
                                       fast_measure=self.fast_measure, ansatz=self.ansatz, out_dim=self.out_dim,
                                       precise=qf.resolve_precise(self.solver_kwargs.get("precise", "auto"), x,
                                                                  self.out_dim)).to(self.p_dtype)
        base = torch.einsum("oi,bi->boi", self._as_oi(self.base_weight), self.base_activation(x))
        return ((postacts + self._as_oi(self.postact_bias)) * self._as_oi(self.postact_weights)[None]
                + base) * self._as_oi(self.mask)[None]

    @torch.no_grad()
    def edge_output_std(self, x: torch.Tensor) -> torch.Tensor:
        """``torch.std(forward_no_sum(x), dim=0)``, shape ``(O, I)``, computed inside the kernels.

        This is the per-edge activation scale the model's ``save_act`` pass needs
        (``src/qkan/qkan.py:1287-1292``); the ``(B, O, I)`` tensor the reference forms for it is never
        allocated. Base activations other than silu are not fused, so they take the ``forward_no_sum`` route.
        """
        assert x.shape[1] == self.in_dim, "Invalid input dimension"
        self._check_solver()
        has_base = self.ba_trainable or self._bw_is_nonzero or bool(self.base_weight.requires_grad)
        if has_base and not isinstance(self.base_activation, nn.SiLU):
            return torch.std(self.forward_no_sum(x), dim=0)
        theta, pw, pb = self._kernel_params()
        mask = None if self._mask_is_identity else self._as_oi(self.mask)
        prep = qf.prepare_layer(theta, pw, pb, self._as_oi(self.postact_weights), None,
                                self._as_oi(self.base_weight) if has_base else None, mask, in_dim=self.in_dim,
                                preact_trainable=self.preact_trainable, fast_measure=self.fast_measure,
                                use_postact_bias=False, ansatz=self.ansatz)
        return qf.edge_stats(prep, x).to(self.p_dtype)

    def get_subset(self, in_id, out_id) -> "QKANLayer":
        """Smaller layer holding the selected input / output neurons (``src/qkan/qkan.py:893-957``)."""
        sub = QKANLayer(len(in_id), len(out_id), reps=self.reps, device=self.device, solver=self.solver,
                        ansatz=self.ansatz, preact_trainable=self.preact_trainable,
                        postact_weight_trainable=self.postact_weight_trainable,
                        postact_bias_trainable=self.postact_bias_trainable,
                        base_activation=self.base_activation, ba_trainable=self.ba_trainable,
                        seed=self.seed, p_dim=self.p_dim)
        pick = lambda t: t.data[out_id][:, in_id]  # noqa: E731
        with torch.no_grad():
            if self._theta_natural().dim() == 4:
                sub._theta_natural().copy_(pick(self._theta_natural()))
                sub._preacts_w_natural().copy_(pick(self._preacts_w_natural()))
                sub._preacts_b_natural().copy_(pick(self._preacts_b_natural()))
            else:
                sub._theta_natural().copy_(self._theta_natural().data)
                sub._preacts_w_natural().copy_(self._preacts_w_natural().data)
                sub._preacts_b_natural().copy_(self._preacts_b_natural().data)
            for name in ("base_weight", "postact_weights", "postact_bias", "mask"):
                sub._as_oi(getattr(sub, name)).copy_(pick(self._as_oi(getattr(self, name))))
            sub._mask_is_identity = bool((sub.mask == 1).all())
            sub._pb_is_nonzero = bool(sub.postact_bias.data.any())
            sub._bw_is_nonzero = bool(sub.ba_trainable or sub.base_weight.data.any())
        return sub
