"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import (GRAD_NAMES, TOL_BF16, TOL_F32, ansatz_case_inputs, case_inputs,
                        expand_group, golden_ansatz_cases, golden_group_cases, golden_layer_cases, nerr,
                        random_problem, reduce_group)

pytestmark = pytest.mark.gpu


def _dev(a, dtype=torch.float32):
    return None if a is None else torch.as_tensor(np.asarray(a), dtype=dtype, device="cuda")


def _run_cuda(p, cfg, io_dtype=torch.float32, param_dtype=torch.float32, precise=False):
    from qkan_b200 import functional as F

    x = _dev(p["x"], io_dtype)
    gy = _dev(p["gy"], io_dtype)
    th, pw, pb = _dev(p["theta"]), _dev(p["pw"]), _dev(p["pb"])
    postw, postb, basew, mask = (_dev(p[k], param_dtype) for k in ("postw", "postb", "basew", "mask"))
    y = F.layer_forward(x, th, pw, pb, postw, postb, basew, mask, precise=precise, **cfg)
    g = F.layer_backward(x, th, pw, pb, postw, postb, basew, mask, gy, precise=precise, **cfg)
    torch.cuda.synchronize()
    return y.float().cpu().numpy(), {k: v.float().cpu().numpy() for k, v in g.items()}


@pytest.mark.parametrize("case", golden_ansatz_cases(), ids=lambda c: c["name"])
def test_golden_rpz_and_real_cases_fp32(case):
    """rpz_encoding and real ansaetze: CUDA fp32 vs the reference's float64 outputs."""
    p = ansatz_case_inputs(case)
    for precise in (False, True):
        y, g = _run_cuda(p, case["cfg"], precise=precise)
        _check(y, g, case["y"], {k: case["g_" + k] for k in GRAD_NAMES}, TOL_F32, case["name"])


@pytest.mark.parametrize("case", golden_group_cases(), ids=lambda c: c["name"])
def test_golden_grouped_parameter_cases_fp32(case):
    """Grouped theta / preacts (g, ...) read in place by the kernels vs the reference's own broadcast."""
    from qkan_b200 import functional as F

    cfg = case["cfg"]
    p = dict(x=case["in_x"], theta=case["in_theta"], pw=case["in_preacts_weight"], pb=case["in_preacts_bias"],
             postw=case["in_postact_weights"], postb=case["in_postact_bias"], basew=None, mask=None,
             gy=case["in_gy"])
    names = [k for k in GRAD_NAMES if k != "base_weight"]
    for precise in (False, True):
        y, g = _run_cuda(p, cfg, precise=precise)
        assert nerr(y, case["y"]) <= TOL_F32
        for k in names:
            assert g[k].shape == case["g_" + k].shape, k
            assert nerr(g[k], case["g_" + k]) <= TOL_F32, f"{case['name']}: grad {k} err {nerr(g[k], case['g_' + k]):.3e}"
    # solver-contract op with the same grouped tensors
    O = case["in_postact_weights"].shape[0]
    x, th, pw, pb = (_dev(p[k]).requires_grad_(True) for k in ("x", "theta", "pw", "pb"))
    pa = F.qkan_postacts(x, th, pw, pb, preact_trainable=cfg["preact_trainable"], fast_measure=cfg["fast_measure"],
                         ansatz=cfg["ansatz"], out_dim=O)
    assert nerr(pa.detach().cpu().numpy(), case["postacts"]) <= TOL_F32
    w = _dev(case["in_postact_weights"]); gy = _dev(case["in_gy"])
    ((pa + _dev(case["in_postact_bias"])) * w).sum(dim=2).mul(gy).sum().backward()
    assert nerr(th.grad.cpu().numpy(), case["g_theta"]) <= TOL_F32
    assert nerr(x.grad.cpu().numpy(), case["g_x"]) <= TOL_F32


def test_grouped_parameters_at_layer_scale_vs_oracle():
    """Group reduction over many outputs and ragged input classes (I = 100 over g = 7), base term and mask on."""
    B, I, O, R, G = 200, 100, 37, 3, 7
    p = random_problem(11, B, I, O, R, use_pb=True, base=True, masked=True)
    rng = np.random.default_rng(5)
    grouped = dict(theta=rng.uniform(-np.pi, np.pi, (G, R + 1, 2)).astype(np.float32),
                   pw=(1 + 0.3 * rng.standard_normal((G, R))).astype(np.float32),
                   pb=(0.3 * rng.standard_normal((G, R))).astype(np.float32))
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True, ansatz="pz_encoding")
    y, g = _run_cuda(dict(p, **grouped), cfg)
    y_ref, g_ref = _run_oracle(dict(p, **{k: expand_group(v, O, I) for k, v in grouped.items()}), cfg)
    for k in ("theta", "preacts_weight", "preacts_bias"):
        g_ref[k] = reduce_group(g_ref[k], G)
    _check(y, g, y_ref, g_ref, TOL_F32, "grouped layer")


@pytest.mark.parametrize("ansatz,B,I,O,R", [("pz", 70, 33, 20, 9), ("pz", 40, 64, 12, 12), ("pz", 33, 20, 9, 16),
                                             ("rpz", 50, 40, 17, 11), ("rpz", 300, 70, 33, 3), ("real", 300, 70, 33, 5),
                                             ("real", 64, 5, 3, 16)])
def test_long_circuits_and_other_ansaetze_vs_oracle(ansatz, B, I, O, R):
    """Repetition counts above 8 run in the padded 12 / 16 instantiations; rpz and real at larger sizes."""
    p = random_problem(B + R, B, I, O, R, use_pb=True, base=True, masked=True)
    layers, width = {"pz": (R + 1, 2), "rpz": (R + 1, 1), "real": (R, 1)}[ansatz]
    rng = np.random.default_rng(R)
    p["theta"] = rng.uniform(-np.pi, np.pi, (O, I, layers, width)).astype(np.float32)
    cfg = dict(preact_trainable=(R % 2 == 1), fast_measure=(R % 3 != 0), use_postact_bias=True, ansatz=ansatz)
    y, g = _run_cuda(p, cfg)
    y_ref, g_ref = _run_oracle(p, cfg)
    _check(y, g, y_ref, g_ref, TOL_F32, f"{ansatz} B{B} I{I} O{O} R{R}")


def _run_oracle(p, cfg):
    args = [p[k] for k in ("x", "theta", "pw", "pb", "postw", "postb", "basew", "mask")]
    y = oracle.forward(*args, **cfg)
    g = oracle.backward(*args, p["gy"], **cfg)
    return y, g


def _check(y, g, y_ref, g_ref, tol, label):
    assert nerr(y, y_ref) <= tol, f"{label}: y err {nerr(y, y_ref):.3e}"
    for k in GRAD_NAMES:
        assert nerr(g[k], g_ref[k]) <= tol, f"{label}: grad {k} err {nerr(g[k], g_ref[k]):.3e}"


@pytest.mark.parametrize("precise", [False, True], ids=["sfu", "precise"])
@pytest.mark.parametrize("case", golden_layer_cases(), ids=lambda c: c["name"])
def test_golden_cases_fp32(case, precise):
    """CUDA fp32 (special-function-unit path and full-precision path) vs the reference's float64 outputs."""
    p = case_inputs(case)
    y, g = _run_cuda(p, case["cfg"], precise=precise)
    g_ref = {k: case["g_" + k] for k in GRAD_NAMES}
    _check(y, g, case["y"], g_ref, TOL_F32 if not precise else 3e-6, case["name"])


@pytest.mark.parametrize("B,I,O,R", [(1, 1, 1, 1), (33, 7, 5, 2), (100, 40, 33, 3), (257, 64, 64, 3),
                                     (64, 300, 9, 4), (50, 31, 70, 8), (1000, 1, 1, 3),
                                     (513, 96, 17, 5), (70, 33, 300, 6), (40, 20, 10, 7)])
@pytest.mark.parametrize("fast", [True, False])
def test_oracle_parity_fp32(B, I, O, R, fast):
    p = random_problem(B * 7 + I + R, B, I, O, R, use_pb=True, base=(R % 2 == 0), masked=(R % 3 == 0))
    cfg = dict(preact_trainable=(O % 2 == 1) or R == 3, fast_measure=fast, use_postact_bias=True)
    y, g = _run_cuda(p, cfg)
    y_ref, g_ref = _run_oracle(p, cfg)
    _check(y, g, y_ref, g_ref, TOL_F32, f"B{B} I{I} O{O} R{R}")


@pytest.mark.parametrize("B,I,O,R", [(64, 64, 48, 1), (129, 96, 64, 2), (200, 128, 40, 4), (96, 70, 33, 8)])
def test_oracle_parity_bf16_io(B, I, O, R):
    """bf16 x / y / grad_y / grad_x and (O,I) tensors, fp32 theta and accumulation (tolerance 2e-2).

    The oracle consumes the bf16-rounded inputs, as the parity protocol prescribes.
    """
    p = random_problem(B + I, B, I, O, R, use_pb=False, x_scale=3.0)
    for k in ("x", "gy", "postw"):
        p[k] = torch.as_tensor(p[k]).to(torch.bfloat16).float().numpy()
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=False)
    y, g = _run_cuda(p, cfg, io_dtype=torch.bfloat16, param_dtype=torch.bfloat16)
    y_ref, g_ref = _run_oracle(p, cfg)
    _check(y, g, y_ref, g_ref, TOL_BF16, f"bf16 B{B} I{I} O{O} R{R}")


def test_postacts_contract_matches_golden():
    """Solver contract: (B,O,I) activations and their backward from a (B,O,I) cotangent."""
    from qkan_b200 import functional as F

    for case in golden_layer_cases():
        p = case_inputs(case)
        cfg = dict(preact_trainable=case["cfg"]["preact_trainable"], fast_measure=case["cfg"]["fast_measure"])
        x, th, pw, pb = (_dev(p[k]) for k in ("x", "theta", "pw", "pb"))
        pa = F.postacts_forward(x, th, pw, pb, **cfg)
        assert nerr(pa.cpu().numpy(), case["postacts"]) <= TOL_F32, case["name"]
        rng = np.random.default_rng(5)
        gpa = rng.standard_normal(case["postacts"].shape).astype(np.float32)
        g = F.postacts_backward(x, th, pw, pb, _dev(gpa), **cfg)
        ref = oracle.backward(p["x"], p["theta"], p["pw"], p["pb"], p["postw"], None, None, None,
                              np.zeros_like(p["gy"]), gpostacts=gpa, use_postact_bias=False, **cfg)
        for k in ("x", "theta", "preacts_weight", "preacts_bias"):
            assert nerr(g[k].cpu().numpy(), ref[k]) <= TOL_F32, (case["name"], k)


def test_backward_is_bitwise_reproducible():
    p = random_problem(3, 300, 70, 50, 3)
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    _, g1 = _run_cuda(p, cfg)
    _, g2 = _run_cuda(p, cfg)
    for k in GRAD_NAMES:
        assert np.array_equal(g1[k], g2[k]), k


def test_empty_batch_and_bad_arguments():
    from qkan_b200 import functional as F

    p = random_problem(1, 4, 3, 2, 2)
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=False)
    th, pw, pb, postw = (_dev(p[k]) for k in ("theta", "pw", "pb", "postw"))
    x0 = torch.empty((0, 3), device="cuda")
    y0 = F.layer_forward(x0, th, pw, pb, postw, **cfg)
    assert y0.shape == (0, 2)
    g0 = F.layer_backward(x0, th, pw, pb, postw, None, None, None, torch.empty((0, 2), device="cuda"), **cfg)
    assert float(g0["theta"].abs().max()) == 0.0
    with pytest.raises(ValueError):
        F.layer_forward(torch.zeros((4, 5), device="cuda"), th, pw, pb, postw, **cfg)
    with pytest.raises(RuntimeError):
        F.layer_forward(torch.zeros((4, 3)), th, pw, pb, postw, **cfg)


def test_c_abi_rejects_bad_workspaces_and_null_pointers():
    """Error behaviour of the raw entry points: negative return code, text in qk_last_error, nothing launched."""
    from qkan_b200 import _abi

    lib = _abi.load()
    desc = _abi.QkDesc(8, 4, 3, 2, _abi.QK_F32, _abi.QK_F32, _abi.QK_FAST_MEASURE, _abi.QK_ANSATZ_PZ)
    dp = _abi.desc_pointer(desc)
    need = lib.qk_forward_workspace_bytes(dp)
    buf = torch.zeros(need + 512, dtype=torch.uint8, device="cuda")
    t = torch.zeros(4096, device="cuda")
    args = [t.data_ptr()] * 5 + [None, None, None, t.data_ptr()]  # x theta pw pb postw | postb basew mask | y
    aligned = (buf.data_ptr() + 255) // 256 * 256
    assert lib.qk_pz_forward(dp, *args, aligned, need - 1, None) == _abi.QK_ERR_WORKSPACE
    assert b"workspace too small" in lib.qk_last_error()
    assert lib.qk_pz_forward(dp, *args, aligned + 4, need, None) == _abi.QK_ERR_WORKSPACE
    assert b"aligned" in lib.qk_last_error()
    assert lib.qk_pz_forward(dp, None, *args[1:], aligned, need, None) == _abi.QK_ERR_BAD_ARGUMENT
    bad = _abi.QkDesc(8, 4, 3, 17, _abi.QK_F32, _abi.QK_F32, 0, _abi.QK_ANSATZ_PZ)
    assert lib.qk_pz_forward(_abi.desc_pointer(bad), *args, aligned, need, None) == _abi.QK_ERR_UNSUPPORTED
    bad = _abi.QkDesc(8, 4, 3, 2, _abi.QK_F32, _abi.QK_F32, 0, 7)
    assert lib.qk_pz_forward(_abi.desc_pointer(bad), *args, aligned, need, None) == _abi.QK_ERR_BAD_ARGUMENT
    assert lib.qk_pz_forward(dp, *args, aligned, need, None) == _abi.QK_OK
    torch.cuda.synchronize()


@pytest.mark.parametrize("x_scale,precise", [(3.0, False), (10.0, False), (10.0, True), (300.0, True)])
def test_accuracy_for_large_input_magnitudes(x_scale, precise):
    """Large |x|: a float32 data angle pw*x + c carries half an ulp of its magnitude, which no float32 path can
    avoid. Up to |x| = 3 everything stays inside 1e-5; beyond, the kernels must be no worse than twice the float32
    build of the CPU restatement (correctly rounded libm sin/cos) on each tensor."""
    p = random_problem(77, 200, 48, 24, 3, use_pb=True, x_scale=x_scale)
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    y, g = _run_cuda(p, cfg, precise=precise)
    y_ref, g_ref = _run_oracle(p, cfg)
    if x_scale <= 3.0:
        _check(y, g, y_ref, g_ref, TOL_F32, f"x_scale {x_scale} precise {precise}")
        return
    args = [p[k] for k in ("x", "theta", "pw", "pb", "postw", "postb", "basew", "mask")]
    y32 = oracle.forward(*args, dtype=np.float32, **cfg)
    g32 = oracle.backward(*args, p["gy"], dtype=np.float32, **cfg)
    assert nerr(y, y_ref) <= max(TOL_F32, 2 * nerr(y32, y_ref))
    for k in GRAD_NAMES:
        bound = max(TOL_F32, 2 * nerr(g32[k], g_ref[k]))
        assert nerr(g[k], g_ref[k]) <= bound, f"x_scale {x_scale} precise {precise}: grad {k} {nerr(g[k], g_ref[k]):.3e} > {bound:.3e}"


@pytest.mark.parametrize("io_dtype,precise", [(torch.float32, False), (torch.float32, True), (torch.bfloat16, False)])
def test_backward_with_sliced_outputs_matches_oracle(io_dtype, precise):
    """Small batches cut the outputs into slices over grid.z and add the grad_x shares afterwards; forced here
    (4 slices of 16, the last one ragged) and compared with the default choice and the oracle."""
    from qkan_b200 import functional as F

    B, I, O, R = 70, 40, 50, 3
    p = random_problem(21, B, I, O, R, use_pb=True, base=True, masked=True)
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    if io_dtype == torch.bfloat16:
        for k in ("x", "gy"):
            p[k] = torch.as_tensor(p[k]).to(torch.bfloat16).float().numpy()
    y_ref, g_ref = _run_oracle(p, cfg)
    tol = TOL_F32 if io_dtype == torch.float32 else TOL_BF16
    from qkan_b200 import _abi

    lib = _abi.load()
    try:
        lib.qk_debug_set(_abi.QK_DBG_BWD_OSPLIT, 4)
        y, g = _run_cuda(p, cfg, io_dtype=io_dtype, precise=precise)
        _check(y, g, y_ref, g_ref, tol, "sliced")
        # solver-contract backward (grad_postacts input) through the same slices
        x, th, pw, pb = (_dev(p[k]) for k in ("x", "theta", "pw", "pb"))
        gpa = torch.randn(B, O, I, device="cuda")
        gs = F.postacts_backward(x, th, pw, pb, gpa, preact_trainable=True, precise=precise)
        lib.qk_debug_set(_abi.QK_DBG_BWD_OSPLIT, 1)
        g1 = F.postacts_backward(x, th, pw, pb, gpa, preact_trainable=True, precise=precise)
    finally:
        lib.qk_debug_set(_abi.QK_DBG_BWD_OSPLIT, 0)
    for k in g1:
        assert nerr(gs[k].cpu().numpy(), g1[k].cpu().numpy()) <= 2e-6, k


def test_seeded_random_shapes_and_flags_vs_oracle():
    """Forty seeded problems over shape, repetitions, ansatz, flags, grouping and dtype: every tile choice
    the dispatcher can make at these sizes (row tiles, output slices, padded circuits) against the oracle."""
    rng = np.random.default_rng(2024)
    for case in range(40):
        ansatz = ("pz", "pz", "rpz", "real")[case % 4]
        B = int(rng.choice([1, 7, 33, 130, 513, 1100]))
        I = int(rng.choice([1, 5, 32, 33, 70, 200]))
        O = int(rng.choice([1, 3, 16, 40, 97, 160]))
        R = int(rng.choice([1, 2, 3, 5, 9]))
        if B * I * O > 6_000_000:
            B = max(1, 6_000_000 // (I * O))
        p = random_problem(1000 + case, B, I, O, R, use_pb=bool(case % 3), base=bool(case % 2), masked=bool(case % 5 == 0))
        layers, width = {"pz": (R + 1, 2), "rpz": (R + 1, 1), "real": (R, 1)}[ansatz]
        group = int(rng.choice([0, 0, 1, 3, 8]))
        lead = (group,) if group else (O, I)
        p["theta"] = rng.uniform(-np.pi, np.pi, lead + (layers, width)).astype(np.float32)
        p["pw"] = (1 + 0.2 * rng.standard_normal(lead + (R,))).astype(np.float32)
        p["pb"] = (0.2 * rng.standard_normal(lead + (R,))).astype(np.float32)
        cfg = dict(preact_trainable=bool(case % 2 == 0), fast_measure=bool(case % 3 != 1),
                   use_postact_bias=p["postb"] is not None, ansatz=ansatz)
        y, g = _run_cuda(p, cfg, precise=bool(case % 7 == 0))
        q = dict(p)
        if group:
            for k in ("theta", "pw", "pb"):
                q[k] = expand_group(p[k], O, I)
        y_ref, g_ref = _run_oracle(q, cfg)
        if group:
            for k in ("theta", "preacts_weight", "preacts_bias"):
                g_ref[k] = reduce_group(g_ref[k], group)
        label = f"case {case}: {ansatz} B{B} I{I} O{O} R{R} group {group} {cfg}"
        assert nerr(y, y_ref) <= TOL_F32, label
        for k in GRAD_NAMES:
            if k == "base_weight" and p["basew"] is None:
                continue
            if k == "postact_bias" and p["postb"] is None:
                continue
            assert nerr(g[k], g_ref[k]) <= TOL_F32, f"{label}: grad {k} err {nerr(g[k], g_ref[k]):.3e}"


@pytest.mark.parametrize("B,I,O,io_dtype", [(19205, 202, 70, torch.float32), (19200, 200, 130, torch.float32),
                                            (19200, 200, 130, torch.bfloat16), (300, 37, 9, torch.float32),
                                            (19200, 200, 128, torch.bfloat16), (300, 40, 12, torch.bfloat16)],
                         ids=["ragged-scalar-columns", "two-output-tiles", "bf16", "small-tiles",
                              "bf16-four-outputs-at-a-time", "bf16-small-tiles"])
def test_base_term_backward_products(B, I, O, io_dtype):
    """The base term's two matrix products (grad_x share and grad_base_weight) at shapes that use the 128-wide
    tiles, several slabs of batch rows, ragged tile edges and both the four-column and the single-column
    epilogue, against the oracle; asking for one of the two results alone runs one kind of CTA only and gives
    the same bits."""
    from qkan_b200 import functional as F

    R = 1
    p = random_problem(B + I + O, B, I, O, R, use_pb=True, base=True, masked=True)
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    bf16 = io_dtype == torch.bfloat16
    if bf16:
        for k in ("x", "gy"):  # the oracle sees the bf16-rounded activations
            p[k] = torch.as_tensor(p[k]).to(torch.bfloat16).float().numpy()
    y, g = _run_cuda(p, cfg, io_dtype=io_dtype)
    y_ref, g_ref = _run_oracle(p, cfg)
    _check(y, g, y_ref, g_ref, TOL_BF16 if bf16 else TOL_F32, f"base term B{B} I{I} O{O}")
    args = [_dev(p["x"], io_dtype)] + [_dev(p[k]) for k in ("theta", "pw", "pb", "postw", "postb", "basew", "mask")]
    for name in ("x", "base_weight"):
        one = F.layer_backward(*args, _dev(p["gy"], io_dtype), want=(name,), **cfg)[name]
        assert np.array_equal(one.float().cpu().numpy(), g[name]), name


def test_grouped_parameters_with_empty_batch_and_bf16():
    """Grouped theta / preacts: an empty batch gives zero gradients in the grouped shapes, and bfloat16
    activations with bfloat16 (O,I) tensors stay inside the bf16 bound against the oracle."""
    from qkan_b200 import functional as F

    B, I, O, R, G = 96, 45, 33, 2, 4
    p = random_problem(9, B, I, O, R, use_pb=True, base=True)
    rng = np.random.default_rng(3)
    p["theta"] = rng.uniform(-np.pi, np.pi, (G, R + 1, 2)).astype(np.float32)
    p["pw"] = (1 + 0.2 * rng.standard_normal((G, R))).astype(np.float32)
    p["pb"] = (0.2 * rng.standard_normal((G, R))).astype(np.float32)
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    th, pw, pb, postw, postb, basew = (_dev(p[k]) for k in ("theta", "pw", "pb", "postw", "postb", "basew"))
    g0 = F.layer_backward(torch.empty((0, I), device="cuda"), th, pw, pb, postw, postb, basew, None,
                          torch.empty((0, O), device="cuda"), **cfg)
    assert g0["theta"].shape == (G, R + 1, 2) and g0["preacts_weight"].shape == (G, R)
    assert all(float(v.abs().max()) == 0.0 for k, v in g0.items() if v.numel())
    for k in ("x", "gy", "postw", "postb", "basew"):  # the oracle sees the bf16-rounded values
        p[k] = torch.as_tensor(p[k]).to(torch.bfloat16).float().numpy()
    y, g = _run_cuda(p, cfg, io_dtype=torch.bfloat16, param_dtype=torch.bfloat16)
    q = dict(p, **{k: expand_group(p[k], O, I) for k in ("theta", "pw", "pb")})
    y_ref, g_ref = _run_oracle(q, cfg)
    for k in ("theta", "preacts_weight", "preacts_bias"):
        g_ref[k] = reduce_group(g_ref[k], G)
    _check(y, g, y_ref, g_ref, TOL_BF16, "grouped bf16")


@pytest.mark.parametrize("frozen,base,io_dtype", [(False, False, torch.float32), (True, True, torch.float32),
                                                  (True, False, torch.bfloat16)])
def test_prepared_entry_points_match_oracle_and_one_call_path(frozen, base, io_dtype):
    """qk_pz_prepare once, then qk_pz_forward_prepared / qk_pz_backward_prepared for two different batches:
    the tables have no batch axis. Results equal the one-call entry points bit for bit (same kernels, same
    tables) and meet the oracle bound; the frozen-preact case carries the second (angle-addition) table."""
    from qkan_b200 import functional as F

    I, O, R = 70, 40, 3
    cfg = dict(preact_trainable=not frozen, fast_measure=True, use_postact_bias=True)
    p = random_problem(31, 150, I, O, R, use_pb=True, base=base, masked=True)
    names = ("theta", "pw", "pb", "postw", "postb", "basew", "mask")
    if io_dtype == torch.bfloat16:
        for k in ("x", "gy"):
            p[k] = torch.as_tensor(p[k]).to(torch.bfloat16).float().numpy()
    dev = {k: (None if p[k] is None else _dev(p[k])) for k in names}
    prep = F.prepare_layer(*(dev[k] for k in names), in_dim=I, **cfg)
    tol = TOL_F32 if io_dtype == torch.float32 else TOL_BF16
    for rows in (150, 37):
        q = dict(p, x=p["x"][:rows], gy=p["gy"][:rows])
        x, gy = _dev(q["x"]).to(io_dtype), _dev(q["gy"]).to(io_dtype)
        y = F.forward_prepared(prep, x)
        g = F.backward_prepared(prep, x, gy)
        y1 = F.layer_forward(x, *(dev[k] for k in names), **cfg)
        g1 = F.layer_backward(x, *(dev[k] for k in names), gy, **cfg)
        assert torch.equal(y, y1)
        for k in g1:
            if k in g:
                assert torch.equal(g[k], g1[k]), k
        y_ref, g_ref = _run_oracle(q, cfg)
        gn = {k: v.float().cpu().numpy() for k, v in g.items()}
        if frozen:
            gn.pop("preacts_weight", None), gn.pop("preacts_bias", None)
        if not base:
            gn.pop("base_weight", None)
        assert nerr(y.float().cpu().numpy(), y_ref) <= tol
        for k, v in gn.items():
            assert nerr(v, g_ref[k]) <= tol, f"rows {rows}: grad {k} {nerr(v, g_ref[k]):.3e}"


def test_prepared_entry_points_reject_short_or_misaligned_buffers():
    from qkan_b200 import _abi

    lib = _abi.load()
    desc = _abi.QkDesc(8, 4, 3, 2, _abi.QK_F32, _abi.QK_F32, _abi.QK_FAST_MEASURE, _abi.QK_ANSATZ_PZ)
    dp = _abi.desc_pointer(desc)
    nt, ns = lib.qk_tables_bytes(dp), lib.qk_backward_scratch_bytes(dp)
    assert nt > 0 and ns > 0 and lib.qk_backward_workspace_bytes(dp) == nt + ns
    assert lib.qk_forward_workspace_bytes(dp) == nt  # frozen preacts: generic table + angle-addition table + bias
    tab = torch.zeros(nt + 512, dtype=torch.uint8, device="cuda")
    t = torch.zeros(4096, device="cuda")
    tp = (tab.data_ptr() + 255) // 256 * 256
    prm = [t.data_ptr()] * 4 + [None, None, None]
    assert lib.qk_pz_prepare(dp, *prm, tp, nt - 1, None) == _abi.QK_ERR_WORKSPACE
    assert lib.qk_pz_prepare(dp, *prm, tp + 8, nt, None) == _abi.QK_ERR_WORKSPACE
    assert lib.qk_pz_prepare(dp, None, *prm[1:], tp, nt, None) == _abi.QK_ERR_BAD_ARGUMENT
    assert lib.qk_pz_prepare(dp, *prm, tp, nt, None) == _abi.QK_OK
    assert lib.qk_pz_forward_prepared(dp, t.data_ptr(), tp, nt - 1, 0, t.data_ptr(), None) == _abi.QK_ERR_WORKSPACE
    assert lib.qk_pz_forward_prepared(dp, t.data_ptr(), tp, nt, 0, None, None) == _abi.QK_ERR_BAD_ARGUMENT
    assert lib.qk_pz_forward_prepared(dp, t.data_ptr(), tp, nt, 0, t.data_ptr(), None) == _abi.QK_OK
    torch.cuda.synchronize()
