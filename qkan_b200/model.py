"""``QKAN``: the reference's model interface (constructor, ``forward``, ``train_``, checkpoints).

Mirrors ``QKAN`` of the reference (``src/qkan/qkan.py:969-2481``) for the parts that are
compute: the constructor and its defaults (``:1022-1065``), the layer stack with the
optional Linear-SiLU-Linear head (``:1170-1211``), ``forward`` (``:1253-1313``),
``train_`` (``:1658-1893``), the activation-scale regulariser it can use
(``:1445-1550``) and rank-0 checkpoint I/O (``:2432-2481``). Plotting, pruning,
attribution and symbolic tooling are not part of this package.
"""
from __future__ import annotations

import os
import random
import warnings
from glob import glob
from typing import Callable, Optional, Union

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from .layer import SOLVER_NAME, QKANLayer, make_base_activation
from .parallel import get_dist_info, print0


class QKANModuleList(nn.ModuleList):
    """Container of the layer stack (``src/qkan/qkan.py:960-966``)."""


class QKAN(nn.Module):
    """Stack of ``QKANLayer`` evaluated by the fused B200 kernels."""

    def __init__(self, width: list, reps: int = 3, group: int = -1, is_map: bool = False,
                 is_batchnorm: bool = False, hidden: int = 0, device="cpu",
                 solver: Union[str, Callable] = SOLVER_NAME, qml_device: str = "default.qubit",
                 ansatz: Union[str, Callable] = "pz_encoding", theta_size: Optional[list] = None,
                 norm_out: int = 0, preact_trainable: bool = False, preact_init: bool = False,
                 postact_weight_trainable: bool = False, postact_bias_trainable: bool = False,
                 base_activation: Union[str, nn.Module] = "silu", ba_trainable: bool = False,
                 fast_measure: bool = True, save_act: bool = False,
                 c_dtype: torch.dtype = torch.complex64, p_dtype: torch.dtype = torch.float32,
                 seed=None, solver_kwargs: Optional[dict] = None, p_dim: int = 4,
                 checkpoint_reps: bool = False, theta_init: str = "xavier", **kwargs):
        super().__init__()
        if seed is not None:
            torch.manual_seed(seed)
            np.random.seed(seed)
            random.seed(seed)
        if p_dim not in (2, 4):
            raise ValueError(f"p_dim must be 2 or 4, got {p_dim}")
        self.depth = len(width) - (2 if is_map else 1)
        self.width, self.reps, self.group, self.device = width, reps, group, device
        self.solver, self.ansatz, self.qml_device = solver, ansatz, qml_device
        self.norm_out = norm_out
        self.postact_weight_trainable = postact_weight_trainable
        self.postact_bias_trainable = postact_bias_trainable
        self.preact_trainable, self.preact_init = preact_trainable, preact_init
        self.theta_size = theta_size
        if isinstance(base_activation, str):
            base_activation = make_base_activation(base_activation)
        self.base_activation = base_activation
        self.ba_trainable, self.fast_measure, self.save_act = ba_trainable, fast_measure, save_act
        self.c_dtype, self.p_dtype, self.seed = c_dtype, p_dtype, seed
        self.solver_kwargs = solver_kwargs or {}
        self.p_dim, self.checkpoint_reps, self.theta_init = p_dim, checkpoint_reps, theta_init

        self.layers = QKANModuleList()
        for l in range(self.depth):
            self.layers.append(QKANLayer(
                in_dim=width[l], out_dim=width[l + 1], reps=reps, group=group, device=device,
                solver=solver, qml_device=qml_device, ansatz=ansatz, theta_size=theta_size,
                preact_trainable=preact_trainable, preact_init=preact_init,
                postact_weight_trainable=postact_weight_trainable,
                postact_bias_trainable=postact_bias_trainable, base_activation=base_activation,
                ba_trainable=ba_trainable, is_batchnorm=is_batchnorm, fast_measure=fast_measure,
                c_dtype=c_dtype, p_dtype=p_dtype, seed=seed, solver_kwargs=self.solver_kwargs,
                p_dim=p_dim, checkpoint_reps=checkpoint_reps, theta_init=theta_init))
        self.is_batchnorm, self.is_map, self.hidden = is_batchnorm, is_map, hidden
        # save_act keeps per-edge STATISTICS (computed inside the kernels). The per-sample edge tensors
        # dr_preacts / dr_postacts of shape (B, O, I) that the reference also stores are only materialised
        # when this is switched on (the plotting tools that read them are not part of this package).
        self.keep_edge_acts = bool(kwargs.get("keep_edge_acts", False))
        if is_map:
            self.layers.append(nn.Linear(width[-2], hidden, device=device, dtype=p_dtype))
            self.layers.append(nn.SiLU())
            self.layers.append(nn.Linear(hidden, width[-1], device=device, dtype=p_dtype))
        self.input_id: Optional[torch.Tensor] = None

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
        for layer in self.layers:
            layer.to(*args, **kwargs)
        return super().to(*args, **kwargs)

    @property
    def param_size(self) -> int:
        total = 0
        for layer in self.layers:
            total += layer.param_size if isinstance(layer, QKANLayer) else sum(
                p.numel() for p in layer.parameters())
        return total

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() not in (2, 3):
            raise NotImplementedError()
        lead = x.shape[:-1]
        x = x.reshape(-1, x.shape[-1])  # a sequence axis is just more batch rows
        rows = x.shape[0]
        if self.input_id is not None:
            x = x[:, self.input_id.long()]
        if self.save_act:
            self.cache_data = x
            self.acts = [x.detach()]
            self.subnode_actscale, self.dr_preacts, self.dr_postacts = [], [], []
            self.acts_scale, self.acts_scale_dr, self.edge_actscale = [], [], []
        for layer in self.layers:
            track = self.save_act and isinstance(layer, QKANLayer)
            if track:
                x_in = x
                self.subnode_actscale.append(torch.std(x, dim=0).detach())
                # per-edge standard deviation over the batch, from the kernels: no (B, O, I) tensor
                output_range = layer.edge_output_std(x)
            x = layer(x)
            if track:
                # every output sees the same inputs, so the (O, I) input range is one row repeated; it keeps
                # its autograd link to the previous layers, as in the reference
                input_range = (torch.std(x_in, dim=0) + 0.1)[None, :].expand(layer.out_dim, layer.in_dim)
                self.edge_actscale.append(output_range)
                self.acts_scale.append((output_range / input_range).detach())
                self.acts_scale_dr.append(output_range / input_range)
                if self.keep_edge_acts:
                    self.dr_preacts.append(x_in.detach()[:, None, :].expand(rows, layer.out_dim, layer.in_dim))
                    self.dr_postacts.append(layer.forward_no_sum(x_in).detach())
                self.acts.append(x.detach())
        if self.norm_out:
            x = F.normalize(x, p=self.norm_out, dim=1)
        return x.reshape(*lead, x.shape[1])

    # ------------------------------------------------------------------ layer extension
    def initialize_parameters(self) -> "QKAN":
        """Reset every QKAN layer in place (theta to zero, the rest to defaults)."""
        for layer in self.layers:
            if isinstance(layer, QKANLayer):
                layer.reset_parameters()
        return self

    def xavier_init(self) -> "QKAN":
        for layer in self.layers:
            if isinstance(layer, QKANLayer):
                layer.xavier_init()
        return self

    def initialize_from_another_model(self, another_model: "QKAN") -> "QKAN":
        """Copy a model with fewer repetitions into this one (``src/qkan/qkan.py:1315-1366``).

        The source's circuit layers fill the leading layers here and the added layers stay at zero
        angles. For pz / rpz the added gates are then Rz rotations in front of a Z readout and zero
        Ry rotations, which leave the readout unchanged: the extended model starts as the same function.
        """
        assert list(self.width) == list(another_model.width), \
            "Cannot initialize from another model with different width"
        linear_src = [m for m in another_model.layers if isinstance(m, nn.Linear)]
        linear_dst = [m for m in self.layers if isinstance(m, nn.Linear)]
        with torch.no_grad():
            for dst, src in zip(self.layers, another_model.layers):
                if not isinstance(dst, QKANLayer):
                    continue
                assert isinstance(src, QKANLayer)
                dst.reset_parameters()
                n_theta = src._theta_natural().shape[-2]
                dst._theta_natural()[..., :n_theta, :].copy_(src._theta_natural())
                dst._preacts_w_natural()[..., : src.reps].copy_(src._preacts_w_natural())
                dst._preacts_b_natural()[..., : src.reps].copy_(src._preacts_b_natural())
                for name in ("postact_weights", "postact_bias", "base_weight"):
                    dst._as_oi(getattr(dst, name)).copy_(src._as_oi(getattr(src, name)))
                dst._pb_is_nonzero = bool(dst.postact_bias.any())
                dst._bw_is_nonzero = bool(dst.ba_trainable or dst.base_weight.any())
            for dst, src in zip(linear_dst, linear_src):
                dst.weight.copy_(src.weight)
                dst.bias.copy_(src.bias)
        return self

    def refine(self, new_reps: int) -> "QKAN":
        """New model with ``new_reps > reps`` repetitions that starts as the same function (layer extension)."""
        assert new_reps > self.reps, "New repetitions must be greater than current repetitions"
        new_model = QKAN(
            width=self.width, reps=new_reps, group=self.group, device=self.device, solver=self.solver,
            qml_device=self.qml_device, ansatz=self.ansatz, theta_size=self.theta_size, norm_out=self.norm_out,
            preact_trainable=self.preact_trainable, preact_init=self.preact_init,
            postact_weight_trainable=self.postact_weight_trainable,
            postact_bias_trainable=self.postact_bias_trainable, base_activation=self.base_activation,
            ba_trainable=self.ba_trainable, is_batchnorm=self.is_batchnorm, is_map=self.is_map,
            hidden=self.hidden, fast_measure=self.fast_measure, save_act=self.save_act, c_dtype=self.c_dtype,
            p_dtype=self.p_dtype, seed=self.seed, solver_kwargs=self.solver_kwargs, p_dim=self.p_dim,
            theta_init=self.theta_init)
        return new_model.initialize_from_another_model(self)

    def layer_extension(self, new_reps: int) -> "QKAN":
        return self.refine(new_reps)

    # ------------------------------------------------------------------ regulariser used by train_
    def get_reg(self, reg_metric: str, lamb_l1: float, lamb_entropy: float, lamb_coef: float,
                lamb_coefdiff: float) -> torch.Tensor:
        """Activation-scale L1 + entropy penalty (``src/qkan/qkan.py:1445-1550``); needs ``save_act``."""
        sources = {"edge_forward_dr_n": "acts_scale_dr", "edge_forward_sum": "acts_scale",
                   "edge_forward_dr_u": "edge_actscale"}
        if reg_metric not in sources:
            if reg_metric in ("edge_backward", "node_backward"):
                raise NotImplementedError(f"reg_metric {reg_metric!r} relies on the attribution tooling, "
                                          "which this package does not include")
            raise RuntimeError(f"reg_metric = {reg_metric} not recognized!")
        reg = torch.tensor(0.0, device=self.device)
        for vec in getattr(self, sources[reg_metric]):
            p_row = vec / (vec.sum(dim=1, keepdim=True) + 1)
            p_col = vec / (vec.sum(dim=0, keepdim=True) + 1)
            ent_row = -torch.mean(torch.sum(p_row * torch.log2(p_row + 1e-4), dim=1))
            ent_col = -torch.mean(torch.sum(p_col * torch.log2(p_col + 1e-4), dim=0))
            reg = reg + lamb_l1 * vec.sum() + lamb_entropy * (ent_row + ent_col)
        for layer in self.layers:
            if isinstance(layer, QKANLayer):
                pw = layer._as_oi(layer.postact_weights)
                reg = reg + lamb_coef * torch.sum(torch.mean(torch.abs(pw), dim=1)) \
                    + lamb_coefdiff * torch.sum(torch.mean(torch.abs(torch.diff(pw)), dim=1))
        return reg

    # ------------------------------------------------------------------ training loop
    def train_(self, dataset, optimizer=None, closure=None, scheduler=None, steps: int = 10, log: int = 1,
               loss_fn=None, batch=-1, lamb=0.0, lamb_l1=1.0, lamb_entropy=2.0, lamb_coef=0.0,
               lamb_coefdiff=0.0, reg_metric="edge_forward_dr_n", verbose=True,
               clip_theta_grad_norm: Optional[float] = None, lamb_theta_l1: float = 0.0,
               prune_every: int = 0, prune_threshold: float = 1e-3):
        """Train on ``dataset`` (keys train_input / train_label / test_input / test_label).

        Same signature, defaults and return value as the reference (``src/qkan/qkan.py:1658-1893``):
        Adam(lr=5e-4) and MSE unless given, LBFGS gets the built-in closure, the result is
        ``{"train_loss": [...], "test_loss": [...], "reg": [...]}`` with one entry per step.
        Under ``torch.distributed`` the gradients are averaged over the ranks after each backward, and the
        objective a closure returns, the logged losses and the value the scheduler sees are means over the ranks,
        so that every rank's optimiser and scheduler take the same decisions (LBFGS line searches included).
        """
        from tqdm import tqdm

        from .parallel import mean_over_ranks, sync_module_grads

        if lamb > 0.0 and not self.save_act:
            lamb = 0.0
            warnings.warn("Regularization is not supported without saving activations", RuntimeWarning)
        loss_fn = loss_fn if loss_fn is not None else torch.nn.MSELoss()
        if optimizer is None:
            optimizer = torch.optim.Adam(self.parameters(), lr=5e-4)
        results: dict = {"train_loss": [], "test_loss": [], "reg": []}
        n_train, n_test = dataset["train_input"].shape[0], dataset["test_input"].shape[0]
        if batch == -1 or batch > n_train:
            batch_size, batch_size_test = n_train, n_test
        else:
            batch_size = batch_size_test = batch
        qkan_layers = [layer for layer in self.layers if isinstance(layer, QKANLayer)]
        theta_params = [layer.theta for layer in qkan_layers]
        state = {"train_loss": None, "reg": None, "train_id": None}

        def objective_and_backward():
            ids = state["train_id"]
            pred = self.forward(dataset["train_input"][ids].to(self.device))
            train_loss = loss_fn(pred, dataset["train_label"][ids].to(self.device))
            if self.save_act:
                reg = self.get_reg(reg_metric, lamb_l1, lamb_entropy, lamb_coef, lamb_coefdiff)
            else:
                reg = torch.tensor(0.0, device=self.device)
            objective = train_loss + lamb * reg
            if lamb_theta_l1 > 0.0:
                objective = objective + lamb_theta_l1 * sum(torch.sum(torch.abs(t)) for t in theta_params)
            objective.backward()
            sync_module_grads(self)
            if clip_theta_grad_norm is not None and theta_params:
                torch.nn.utils.clip_grad_norm_(theta_params, max_norm=clip_theta_grad_norm)
            # Every rank hands its optimiser the same objective (the mean over the row shards, matching the
            # averaged gradients): closure-driven optimisers choose their next collective from this value.
            state["train_loss"], state["reg"] = mean_over_ranks(train_loss), mean_over_ranks(reg)
            return mean_over_ranks(objective)

        def default_closure():
            optimizer.zero_grad()
            return objective_and_backward()

        # closure-driven optimisers: torch's LBFGS, and composites that hand the closure on to one (the
        # reference's LBFGSFinisher, src/qkan/optim/lbfgs.py:46-130, or anything that sets `needs_closure`)
        is_lbfgs = (isinstance(optimizer, torch.optim.LBFGS) or bool(getattr(optimizer, "needs_closure", False))
                    or type(optimizer).__name__ == "LBFGSFinisher")
        if closure is None and is_lbfgs:
            closure = default_closure

        pbar = tqdm(range(steps), ncols=100, disable=not verbose)
        for step in pbar:
            self.train()
            state["train_id"] = np.random.choice(n_train, batch_size, replace=False)
            test_id = np.random.choice(n_test, batch_size_test, replace=False)
            if is_lbfgs:
                optimizer.step(closure)
            else:
                optimizer.zero_grad()
                objective_and_backward()
                optimizer.step(closure)
            if prune_every > 0 and (step + 1) % prune_every == 0:
                with torch.no_grad():
                    for layer in qkan_layers:
                        kill = torch.sum(torch.abs(layer._theta_natural()), dim=(-2, -1)) < prune_threshold
                        mask_2d = layer._as_oi(layer.mask).data
                        if not bool(kill.any()) or kill.numel() != mask_2d.numel():
                            continue  # grouped theta has no per-edge magnitude
                        mask_2d[kill.reshape(mask_2d.shape)] = 0.0
                        layer._mask_is_identity = False
            self.eval()
            with torch.no_grad():
                test_loss = loss_fn(self.forward(dataset["test_input"][test_id].to(self.device)),
                                    dataset["test_label"][test_id].to(self.device))
            test_loss = mean_over_ranks(test_loss)  # one value for every rank's scheduler
            if scheduler is not None:
                scheduler.step(test_loss)
            train_loss = state["train_loss"]
            if verbose and step % log == 0:
                pbar.set_postfix({"train loss": float(train_loss), "test loss": float(test_loss)})
            results["train_loss"].append(train_loss.detach().cpu().numpy())
            results["test_loss"].append(test_loss.detach().cpu().numpy())
            results["reg"].append(state["reg"].detach().cpu().numpy())
        return results

    # ------------------------------------------------------------------ checkpoints (rank 0 writes)
    @staticmethod
    def clear_ckpts(folder="./model_ckpt"):
        is_ddp, rank, _, _ = get_dist_info()
        if not is_ddp or rank == 0:
            if os.path.exists(folder):
                for f in glob(folder + "/*"):
                    os.remove(f)
            else:
                os.makedirs(folder)

    def save_ckpt(self, name, folder="./model_ckpt"):
        is_ddp, rank, _, _ = get_dist_info()
        if not is_ddp or rank == 0:
            os.makedirs(folder, exist_ok=True)
            torch.save(self.state_dict(), folder + "/" + name)
            print0("save this model to", folder + "/" + name)

    def load_ckpt(self, name, folder="./model_ckpt"):
        self.load_state_dict(torch.load(folder + "/" + name))
