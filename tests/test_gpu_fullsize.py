"""Parity at the benchmark configurations' full sizes, through sampled rows / edges and size-independent properties.

The oracle cannot evaluate 4e9 edges, but every output has a small dependency cone:
``y[b,:]`` and ``grad_x[b,:]`` depend on row ``b`` only, and the parameter gradients of edge
``(o,i)`` depend on column ``i`` of ``x`` and column ``o`` of ``grad_y`` only. So random rows and
random edges of the full-size CUDA result are compared with the oracle run on exactly those
cones, and linearity / additivity of the backward cover the rest.
"""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import TOL_BF16, TOL_F32, nerr

pytestmark = pytest.mark.gpu

PARAM_GRADS = ("theta", "preacts_weight", "preacts_bias", "postact_weights", "postact_bias")


def _problem(seed, B, I, O, R, io_dtype, x_kind, trainable=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rand = lambda *s: torch.rand(*s, generator=g, device="cuda")  # noqa: E731
    randn = lambda *s: torch.randn(*s, generator=g, device="cuda")  # noqa: E731
    x = rand(B, I) * 2 - 1 if x_kind == "uniform" else randn(B, I).clamp_(-3, 3)
    p = dict(
        x=x.to(io_dtype), theta=(rand(O, I, R + 1, 2) * 2 - 1) * np.pi,
        pw=1 + 0.1 * randn(O, I, R) if trainable else torch.ones(O, I, R, device="cuda"),
        pb=0.1 * randn(O, I, R) if trainable else torch.zeros(O, I, R, device="cuda"),
        postw=(randn(O, I) / np.sqrt(I)).to(io_dtype), postb=(0.1 * randn(O, I)).to(io_dtype),
        gy=randn(B, O).to(io_dtype))
    return p


def _run(p, cfg):
    from qkan_b200 import functional as F

    y = F.layer_forward(p["x"], p["theta"], p["pw"], p["pb"], p["postw"], p["postb"], None, None, **cfg)
    g = F.layer_backward(p["x"], p["theta"], p["pw"], p["pb"], p["postw"], p["postb"], None, None,
                         p["gy"], **cfg)
    torch.cuda.synchronize()
    return y, g


def _np(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def _check_sampled(p, cfg, y, g, tol, n_rows, n_edges, seed=0):
    rng = np.random.default_rng(seed)
    B, I = p["x"].shape
    O = p["theta"].shape[0]
    rows = np.sort(rng.choice(B, size=min(n_rows, B), replace=False))
    par = [_np(p[k]) for k in ("theta", "pw", "pb", "postw", "postb")]
    xr, gyr = _np(p["x"][rows]), _np(p["gy"][rows])
    y_ref = oracle.forward(xr, *par, None, None, **cfg)
    g_ref = oracle.backward(xr, *par, None, None, gyr, **cfg)
    scale_y = float(np.abs(_np(y)).max())
    scale_gx = float(np.abs(_np(g["x"])).max())
    assert np.abs(_np(y[rows]) - y_ref).max() <= tol * scale_y
    assert np.abs(_np(g["x"][rows]) - g_ref["x"]).max() <= tol * scale_gx
    # parameter gradients of random edges over the FULL batch
    xs, gys = _np(p["x"]), _np(p["gy"])
    scales = {k: float(np.abs(_np(g[k])).max()) for k in PARAM_GRADS}
    for _ in range(n_edges):
        o, i = int(rng.integers(O)), int(rng.integers(I))
        sub = [a[o:o + 1, i:i + 1] for a in par]
        ref = oracle.backward(xs[:, i:i + 1], *sub, None, None, gys[:, o:o + 1], **cfg)
        for k in PARAM_GRADS:
            got = _np(g[k][o, i])
            assert np.abs(got - ref[k][0, 0]).max() <= tol * scales[k], (k, o, i)


def test_layer_microbenchmark_full_size_fp32():
    """Batch 65536, 256 -> 256, reps 3, float32 (the headline configuration)."""
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    p = _problem(0, 65536, 256, 256, 3, torch.float32, "uniform")
    y, g = _run(p, cfg)
    _check_sampled(p, cfg, y, g, TOL_F32, n_rows=48, n_edges=12)
    # the backward is linear in grad_y: scaling by 2 is exact in binary floating point
    p2 = dict(p, gy=p["gy"] * 2)
    _, g2 = _run(p2, cfg)
    for k in ("x",) + PARAM_GRADS:
        assert torch.equal(g2[k], g[k] * 2), k
    # additivity over the batch: the two halves sum to the whole
    half = 65536 // 2
    parts = []
    for sl in (slice(0, half), slice(half, None)):
        ph = dict(p, x=p["x"][sl].contiguous(), gy=p["gy"][sl].contiguous())
        yh, gh = _run(ph, cfg)
        assert nerr(_np(yh), _np(y[sl])) <= 1e-6
        assert nerr(_np(gh["x"]), _np(g["x"][sl])) <= 1e-6
        parts.append(gh)
    for k in PARAM_GRADS:
        assert nerr(_np(parts[0][k] + parts[1][k]), _np(g[k])) <= 2e-6, k


@pytest.mark.parametrize("dim,reps", [(512, 1), (512, 4), (512, 8), (1024, 2), (2048, 2)])
def test_bf16_layer_sweep_shapes(dim, reps):
    """Batch 8192, square layers, bf16 x / y / grads and postact weights, fp32 theta and accumulation."""
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    p = _problem(dim + reps, 8192, dim, dim, reps, torch.bfloat16, "normal")
    y, g = _run(p, cfg)
    assert y.dtype == torch.bfloat16 and g["x"].dtype == torch.bfloat16
    _check_sampled(p, cfg, y, g, TOL_BF16, n_rows=4 if dim > 512 else 8, n_edges=6)


def test_mnist_shaped_first_layer_and_hqkan_shaped_layer():
    """784 -> 128 reps 3 fp32 at batch 1024 (default frozen preacts), and 768 -> 768 reps 2 bf16 at 8192 rows."""
    cfg = dict(preact_trainable=False, fast_measure=True, use_postact_bias=True)
    p = _problem(5, 1024, 784, 128, 3, torch.float32, "uniform", trainable=False)
    p["x"] = (p["x"] + 1) / 2  # pixels in [0,1]
    y, g = _run(p, cfg)
    _check_sampled(p, cfg, y, g, TOL_F32, n_rows=16, n_edges=8)
    assert float(g["preacts_weight"].abs().max()) == 0.0
    p = _problem(6, 8192, 768, 768, 2, torch.bfloat16, "normal", trainable=False)
    y, g = _run(p, cfg)
    _check_sampled(p, cfg, y, g, TOL_BF16, n_rows=4, n_edges=6)


def test_mnist_shaped_classifier_trains():
    """QKAN [784,128,10], reps 3, Adam lr 1e-3 on synthetic images: a few steps lower the cross-entropy."""
    from qkan_b200 import QKAN

    torch.manual_seed(0)
    model = QKAN([784, 128, 10], reps=3, seed=0).to("cuda")
    x = torch.rand(1024, 784, device="cuda")
    labels = torch.randint(0, 10, (1024,), device="cuda")
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x), labels)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert np.isfinite(losses).all() and losses[-1] < losses[0]
