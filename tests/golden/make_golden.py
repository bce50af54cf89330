"""Generate the golden fixtures in this directory by running the reference itself.

Usage (only where the reference checkout is mounted; the fixtures are committed so
nothing at test time needs it):

    python tests/golden/make_golden.py /path/to/reference [layer|ansatz|group|init|fit|act]

The reference package imports ``matplotlib`` unconditionally (``src/qkan/qkan.py:33``)
for its plotting helpers; an empty stand-in module is registered before the import,
which does not touch any arithmetic.

What is written:

* ``layer_cases.npz`` — for a grid of small ``QKANLayer`` configurations run with the
  reference ``exact`` solver in complex128/float64: the inputs, ``y``, the per-edge
  ``postacts`` and every gradient of ``sum(y * gy)`` from torch autograd; plus ``y`` from
  the reference's default complex64/float32 arithmetic.
* ``ansatz_cases.npz`` — the same for the ``rpz_encoding`` and ``real`` ansaetze, with the solver called
  directly in float64 (the reference layer forces bfloat16 arithmetic for ``real``, ``qkan.py:272-274``)
  and the epilogue of ``qkan.py:776-785`` applied on top.
* ``init_cases.npz`` — seeded parameter initialisations (``state_dict`` tensors).
* ``fit_case.npz`` — the 1-D function-fit configuration: dataset, seeded initial
  prediction / loss / gradients, and the LBFGS loss trajectory of the reference.
* ``act_cases.npz`` — ``save_act`` statistics of small models (per-layer ``acts_scale``, ``edge_actscale``,
  ``subnode_actscale``) and the regulariser ``get_reg`` built from them.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# name, B, I, O, R, preact_trainable, fast_measure, postact_bias, base, masked
LAYER_CASES = [
    ("tiny_1x1", 9, 1, 1, 3, True, True, True, True, False),
    ("r1_fast", 5, 3, 4, 1, True, True, False, False, False),
    ("r2_born", 6, 4, 3, 2, True, False, True, False, False),
    ("r3_fixed_preact", 7, 5, 2, 3, False, True, False, True, False),
    ("r3_all", 8, 3, 5, 3, True, True, True, True, True),
    ("r4_fixed_born", 4, 2, 3, 4, False, False, True, False, True),
    ("r8_fast", 3, 2, 2, 8, True, True, False, False, False),
    ("wide_in", 4, 37, 3, 2, True, True, True, False, True),
    ("wide_out", 4, 3, 41, 2, False, True, False, True, False),
    ("r5_mixed", 5, 6, 7, 5, True, True, True, True, True),
]


def _import_reference(ref_root: str):
    for name in ("matplotlib", "matplotlib.pyplot"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import qkan  # noqa: F401

    return qkan


def layer_cases(qkan, torch):
    out = {}
    for idx, (name, B, I, O, R, ptr, fast, use_pb, base, masked) in enumerate(LAYER_CASES):
        g = torch.Generator().manual_seed(1000 + idx)
        rnd = lambda *s: torch.rand(*s, generator=g, dtype=torch.float64)  # noqa: E731
        nrm = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)  # noqa: E731
        inp = {
            "x": rnd(B, I) * 4 - 2,
            "theta": (rnd(O, I, R + 1, 2) * 2 - 1) * np.pi,
            "preacts_weight": 1 + 0.3 * nrm(O, I, R),
            "preacts_bias": 0.3 * nrm(O, I, R),
            "postact_weights": nrm(O, I) / np.sqrt(I),
            "postact_bias": 0.5 * nrm(O, I) if use_pb else torch.zeros(O, I, dtype=torch.float64),
            "base_weight": 0.5 * nrm(O, I) if base else torch.zeros(O, I, dtype=torch.float64),
            "mask": (rnd(O, I) > 0.3).double() if masked else torch.ones(O, I, dtype=torch.float64),
            "gy": nrm(B, O),
        }
        flags = dict(preact_trainable=ptr, fast_measure=fast, use_postact_bias=use_pb, base=base,
                     masked=masked)
        for prec, cd, pd in (("f64", torch.complex128, torch.float64), ("f32", torch.complex64, torch.float32)):
            layer = qkan.QKANLayer(I, O, reps=R, solver="exact", preact_trainable=ptr,
                                   postact_weight_trainable=True, postact_bias_trainable=use_pb,
                                   ba_trainable=base, fast_measure=fast, c_dtype=cd, p_dtype=pd)
            with torch.no_grad():
                for pname in ("theta", "preacts_weight", "preacts_bias", "postact_weights",
                              "postact_bias", "base_weight", "mask"):
                    getattr(layer, pname).data.copy_(inp[pname].to(pd))
            layer._mask_is_identity = not masked
            layer.train()
            x = inp["x"].to(pd).clone().requires_grad_(True)
            y = layer(x)
            if prec == "f32":
                out[f"{name}/y_f32"] = y.detach().numpy()
                continue
            (y * inp["gy"]).sum().backward()
            out[f"{name}/y"] = y.detach().numpy()
            solver = qkan.solver.get_solver("exact")
            with torch.no_grad():
                pa = solver(x.detach(), layer.theta, layer.preacts_weight, layer.preacts_bias, R,
                            ansatz="pz_encoding", preacts_trainable=ptr, fast_measure=fast,
                            out_dim=O, dtype=cd)
            out[f"{name}/postacts"] = pa.numpy()
            out[f"{name}/g_x"] = x.grad.numpy()
            for pname in ("theta", "preacts_weight", "preacts_bias", "postact_weights",
                          "postact_bias", "base_weight"):
                grad = getattr(layer, pname).grad
                out[f"{name}/g_{pname}"] = (grad.numpy() if grad is not None
                                            else np.zeros(tuple(getattr(layer, pname).shape)))
        for k, v in inp.items():
            out[f"{name}/in_{k}"] = v.numpy()
        out[f"{name}/flags"] = np.array([int(flags[k]) for k in
                                         ("preact_trainable", "fast_measure", "use_postact_bias",
                                          "base", "masked")], dtype=np.int64)
        out[f"{name}/dims"] = np.array([B, I, O, R], dtype=np.int64)
    out["names"] = np.array([c[0] for c in LAYER_CASES])
    np.savez_compressed(os.path.join(HERE, "layer_cases.npz"), **out)


# name, ansatz, B, I, O, R, preact_trainable, fast_measure
ANSATZ_CASES = [
    ("rpz_r1_fast", "rpz_encoding", 6, 3, 4, 1, True, True),
    ("rpz_r3_fixed", "rpz_encoding", 5, 4, 3, 3, False, True),
    ("rpz_r2_born", "rpz_encoding", 7, 2, 5, 2, True, False),
    ("rpz_r5_wide", "rpz_encoding", 4, 35, 3, 5, True, True),
    ("real_r1_fast", "real", 6, 3, 4, 1, True, True),
    ("real_r2_fixed", "real", 5, 4, 3, 2, False, True),
    ("real_r4_born", "real", 7, 2, 5, 4, True, False),
    ("real_r3_wide", "real", 4, 35, 3, 3, False, False),
]


def ansatz_cases(qkan, torch):
    out = {}
    solver = qkan.solver.get_solver("exact")
    for idx, (name, ansatz, B, I, O, R, ptr, fast) in enumerate(ANSATZ_CASES):
        g = torch.Generator().manual_seed(2000 + idx)
        rnd = lambda *s: torch.rand(*s, generator=g, dtype=torch.float64)  # noqa: E731
        nrm = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)  # noqa: E731
        is_real = ansatz == "real"
        th_shape = (O, I, R, 1) if is_real else (O, I, R + 1, 1)
        leaf = lambda t: t.clone().requires_grad_(True)  # noqa: E731
        x = leaf(rnd(B, I) * 4 - 2)
        theta = leaf((rnd(*th_shape) * 2 - 1) * np.pi)
        pw = leaf(1 + 0.3 * nrm(O, I, R))
        pb = leaf(0.3 * nrm(O, I, R))
        postw = leaf(nrm(O, I) / np.sqrt(I))
        postb = leaf(0.5 * nrm(O, I))
        basew = leaf(0.5 * nrm(O, I))
        mask = (rnd(O, I) > 0.3).double()
        gy = nrm(B, O)
        pa = solver(x, theta, pw, pb, R, ansatz=ansatz, preacts_trainable=ptr, fast_measure=fast,
                    out_dim=O, dtype=torch.float64 if is_real else torch.complex128)
        y = ((pa + postb) * (postw * mask)).sum(dim=2) + torch.nn.functional.silu(x) @ (basew * mask).T
        (y * gy).sum().backward()
        zero = lambda t: t.grad if t.grad is not None else torch.zeros_like(t)  # noqa: E731
        for k, v in dict(in_x=x, in_theta=theta, in_preacts_weight=pw, in_preacts_bias=pb,
                         in_postact_weights=postw, in_postact_bias=postb, in_base_weight=basew,
                         in_mask=mask, in_gy=gy, y=y, postacts=pa, g_x=zero(x), g_theta=zero(theta),
                         g_preacts_weight=zero(pw), g_preacts_bias=zero(pb), g_postact_weights=zero(postw),
                         g_postact_bias=zero(postb), g_base_weight=zero(basew)).items():
            out[f"{name}/{k}"] = v.detach().numpy()
        out[f"{name}/flags"] = np.array([int(ptr), int(fast)], dtype=np.int64)
        out[f"{name}/ansatz"] = np.array(ansatz)
    out["names"] = np.array([c[0] for c in ANSATZ_CASES])
    np.savez_compressed(os.path.join(HERE, "ansatz_cases.npz"), **out)


# name, ansatz, B, I, O, R, group, preact_trainable, fast_measure
GROUP_CASES = [
    ("group_pz_g3", "pz_encoding", 6, 7, 4, 2, 3, True, True),      # 7 inputs over 3 entries: ragged classes
    ("group_pz_g1_fixed", "pz_encoding", 5, 4, 3, 3, 1, False, False),
    ("group_pz_g40_wide", "pz_encoding", 4, 35, 3, 1, 40, True, True),  # more entries than inputs
    ("group_rpz_g2", "rpz_encoding", 5, 5, 2, 2, 2, False, True),
    ("group_real_g3", "real", 6, 8, 3, 3, 3, True, True),
]


def group_cases(qkan, torch):
    """Grouped theta / preacts (g, ...) through the reference solver, which broadcasts them itself."""
    out = {}
    solver = qkan.solver.get_solver("exact")
    for idx, (name, ansatz, B, I, O, R, G, ptr, fast) in enumerate(GROUP_CASES):
        g = torch.Generator().manual_seed(3000 + idx)
        rnd = lambda *s: torch.rand(*s, generator=g, dtype=torch.float64)  # noqa: E731
        nrm = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)  # noqa: E731
        leaf = lambda t: t.clone().requires_grad_(True)  # noqa: E731
        th_shape = {"pz_encoding": (G, R + 1, 2), "rpz_encoding": (G, R + 1, 1), "real": (G, R, 1)}[ansatz]
        x = leaf(rnd(B, I) * 4 - 2)
        theta = leaf((rnd(*th_shape) * 2 - 1) * np.pi)
        pw = leaf(1 + 0.3 * nrm(G, R))
        pb = leaf(0.3 * nrm(G, R))
        postw = leaf(nrm(O, I) / np.sqrt(I))
        postb = leaf(0.5 * nrm(O, I))
        gy = nrm(B, O)
        pa = solver(x, theta, pw, pb, R, ansatz=ansatz, preacts_trainable=ptr, fast_measure=fast,
                    out_dim=O, dtype=torch.float64 if ansatz == "real" else torch.complex128)
        y = ((pa + postb) * postw).sum(dim=2)
        (y * gy).sum().backward()
        zero = lambda t: t.grad if t.grad is not None else torch.zeros_like(t)  # noqa: E731
        for k, v in dict(in_x=x, in_theta=theta, in_preacts_weight=pw, in_preacts_bias=pb,
                         in_postact_weights=postw, in_postact_bias=postb, in_gy=gy, y=y, postacts=pa,
                         g_x=zero(x), g_theta=zero(theta), g_preacts_weight=zero(pw), g_preacts_bias=zero(pb),
                         g_postact_weights=zero(postw), g_postact_bias=zero(postb)).items():
            out[f"{name}/{k}"] = v.detach().numpy()
        out[f"{name}/flags"] = np.array([int(ptr), int(fast)], dtype=np.int64)
        out[f"{name}/ansatz"] = np.array(ansatz)
    out["names"] = np.array([c[0] for c in GROUP_CASES])
    np.savez_compressed(os.path.join(HERE, "group_cases.npz"), **out)


def init_cases(qkan, torch):
    out = {}
    specs = {
        "fit_1_1": dict(width=[1, 1], reps=3, seed=0),
        "mlp_3_4_2": dict(width=[3, 4, 2], reps=2, seed=7, preact_trainable=True, preact_init=True),
        "pdim2": dict(width=[5, 3], reps=3, seed=3, p_dim=2, ba_trainable=True),
        "map_head": dict(width=[4, 3, 6, 2], reps=1, seed=11, is_map=True, hidden=6),
        "bn_small_gauss": dict(width=[3, 2], reps=2, seed=5, is_batchnorm=True, theta_init="small_gaussian"),
    }
    for name, kw in specs.items():
        model = qkan.QKAN(**kw)
        for k, v in model.state_dict().items():
            out[f"{name}/{k}"] = v.detach().numpy()
    layer = qkan.QKANLayer(4, 3, reps=2, seed=1)
    for k, v in layer.state_dict().items():
        out[f"layer_4_3/{k}"] = v.detach().numpy()
    np.savez_compressed(os.path.join(HERE, "init_cases.npz"), **out)


def fit_case(qkan, torch):
    f = lambda x: torch.sin(20 * x) / (20 * x)  # noqa: E731
    dataset = qkan.create_dataset(f, n_var=1, ranges=[0, 1], train_num=1000, test_num=1000, seed=0)
    out = {k: v.numpy() for k, v in dataset.items()}
    for tag, ba in (("ba", True), ("noba", False)):
        model = qkan.QKAN([1, 1], reps=3, seed=0, preact_trainable=True, postact_weight_trainable=True,
                          postact_bias_trainable=True, ba_trainable=ba)
        model.train()
        pred = model(dataset["train_input"])
        loss = torch.nn.functional.mse_loss(pred, dataset["train_label"])
        loss.backward()
        out[f"{tag}/pred0"] = pred.detach().numpy()
        out[f"{tag}/loss0"] = np.array(loss.item())
        for k, p in model.named_parameters():
            if p.grad is not None:
                out[f"{tag}/grad/{k}"] = p.grad.numpy().copy()
        model.zero_grad()
        opt = torch.optim.LBFGS(model.parameters(), lr=5e-2)
        res = model.train_(dataset, optimizer=opt, steps=100, verbose=False)
        out[f"{tag}/train_loss"] = np.array([float(v) for v in res["train_loss"]])
        out[f"{tag}/test_loss"] = np.array([float(v) for v in res["test_loss"]])
    np.savez_compressed(os.path.join(HERE, "fit_case.npz"), **out)


def act_cases(qkan, torch):
    """save_act statistics of the reference's QKAN.forward (src/qkan/qkan.py:1280-1302) and its regulariser
    (src/qkan/qkan.py:1445-1550): the model's state, the input, and per layer acts_scale / edge_actscale /
    subnode_actscale, plus get_reg for the three forward metrics."""
    out = {}
    specs = {
        "mlp_base": dict(width=[5, 4, 3], reps=2, seed=3, ba_trainable=True, save_act=True),
        "mlp_trainable": dict(width=[6, 3, 2], reps=3, seed=5, preact_trainable=True, preact_init=True,
                              postact_weight_trainable=True, postact_bias_trainable=True, save_act=True),
        "born_nobase": dict(width=[4, 5], reps=1, seed=9, fast_measure=False, save_act=True),
    }
    for name, kw in specs.items():
        model = qkan.QKAN(**kw)
        g = torch.Generator().manual_seed(77)
        with torch.no_grad():  # make the (O,I) epilogue tensors non-trivial
            for layer in model.layers:
                layer.postact_weights.add_(0.3 * torch.randn(layer.postact_weights.shape, generator=g))
                layer.postact_bias.add_(0.2 * torch.randn(layer.postact_bias.shape, generator=g))
                layer._pb_is_nonzero = True
        x = torch.rand(64, kw["width"][0], generator=g) * 2 - 1
        y = model(x)
        out[f"{name}/x"] = x.numpy()
        out[f"{name}/y"] = y.detach().numpy()
        for k, v in model.state_dict().items():
            out[f"{name}/state/{k}"] = v.detach().numpy()
        for l in range(len(model.acts_scale)):
            out[f"{name}/acts_scale/{l}"] = model.acts_scale[l].detach().numpy()
            out[f"{name}/edge_actscale/{l}"] = model.edge_actscale[l].detach().numpy()
            out[f"{name}/subnode_actscale/{l}"] = model.subnode_actscale[l].detach().numpy()
        for metric in ("edge_forward_dr_n", "edge_forward_sum", "edge_forward_dr_u"):
            out[f"{name}/reg/{metric}"] = np.array(float(model.get_reg(metric, 1.0, 2.0, 0.1, 0.05)))
    out["names"] = np.array(list(specs))
    np.savez_compressed(os.path.join(HERE, "act_cases.npz"), **out)


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QKAN_REFERENCE_ROOT", "")
    if not ref_root or not os.path.isdir(ref_root):
        raise SystemExit("usage: make_golden.py <reference checkout>")
    import torch

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    qkan = _import_reference(ref_root)
    only = sys.argv[2] if len(sys.argv) > 2 else "all"
    if only in ("all", "layer"):
        layer_cases(qkan, torch)
    if only in ("all", "ansatz"):
        ansatz_cases(qkan, torch)
    if only in ("all", "group"):
        group_cases(qkan, torch)
    if only in ("all", "init"):
        init_cases(qkan, torch)
    if only in ("all", "fit"):
        fit_case(qkan, torch)
    if only in ("all", "act"):
        act_cases(qkan, torch)
    print("wrote", sorted(p for p in os.listdir(HERE) if p.endswith(".npz")))


if __name__ == "__main__":
    main()
