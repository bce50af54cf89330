"""The allocation-free forward entry point, called through the C ABI.

Some hosts of this library cannot allocate device memory at call time (their memory
belongs to another runtime's pool, or cudaMalloc is banned inside their serving loop),
so ``qk_pz_forward_noalloc`` keeps its scratch in an array built into the library.
This file is collected last on purpose: a run that stops at the first failure has then
already exercised every other test.
"""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import TOL_BF16, TOL_F32, nerr, random_problem

pytestmark = pytest.mark.gpu


def _call_both(p, cfg_flags, io_dtype=torch.float32, device_index=0):
    from qkan_b200 import _abi

    lib = _abi.load()
    dev = torch.device("cuda", device_index)
    torch.cuda.set_device(dev)
    t = {k: (None if v is None else torch.from_numpy(v).to(dev)) for k, v in p.items()}
    t["x"] = t["x"].to(io_dtype)
    B, I = p["x"].shape
    O, _, R1, _ = p["theta"].shape
    desc = _abi.QkDesc(B, I, O, R1 - 1, _abi.QK_BF16 if io_dtype == torch.bfloat16 else _abi.QK_F32, _abi.QK_F32,
                       cfg_flags, 0)
    dp = _abi.desc_pointer(desc)
    ptr = lambda k: None if t[k] is None else t[k].data_ptr()  # noqa: E731
    stream = torch.cuda.current_stream(dev).cuda_stream
    # existing entry point with a caller-owned workspace
    nbytes = lib.qk_forward_workspace_bytes(dp)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    y_ref = torch.empty((B, O), device=dev, dtype=io_dtype)
    rc = lib.qk_pz_forward(dp, ptr("x"), ptr("theta"), ptr("pw"), ptr("pb"), ptr("postw"), ptr("postb"),
                           ptr("basew"), ptr("mask"), y_ref.data_ptr(), ws.data_ptr(), nbytes, stream)
    assert rc == 0, _abi.last_error()
    # new entry point: no workspace argument at all
    y = torch.empty((B, O), device=dev, dtype=io_dtype)
    rc = lib.qk_pz_forward_noalloc(dp, ptr("x"), ptr("theta"), ptr("pw"), ptr("pb"), ptr("postw"),
                                   ptr("postb"), ptr("basew"), ptr("mask"), y.data_ptr(), stream)
    assert rc == 0, lib.qk_noalloc_last_error().decode()
    torch.cuda.synchronize()
    return y.float().cpu().numpy(), y_ref.float().cpu().numpy()


def _oracle_y(p, flags):
    from qkan_b200 import _abi

    return oracle.forward(p["x"], p["theta"], p["pw"], p["pb"], p["postw"], p["postb"], p["basew"], p["mask"],
                          preact_trainable=bool(flags & _abi.QK_PREACT_TRAINABLE),
                          fast_measure=bool(flags & _abi.QK_FAST_MEASURE),
                          use_postact_bias=bool(flags & _abi.QK_USE_POSTACT_BIAS))


def test_noalloc_forward_matches_workspace_forward_twice_in_a_row():
    from qkan_b200 import _abi

    flags = _abi.QK_PREACT_TRAINABLE | _abi.QK_FAST_MEASURE | _abi.QK_USE_POSTACT_BIAS
    # two calls in a row with different shapes and values: the second sees the first one's leftovers
    for seed, (B, I, O, R) in enumerate([(130, 70, 40, 3), (64, 33, 90, 2)]):
        p = random_problem(50 + seed, B, I, O, R, use_pb=True, base=(seed == 1), masked=True)
        y, y_ref = _call_both(p, flags)
        assert np.isfinite(y).all()
        assert nerr(y, y_ref) <= TOL_F32, f"call {seed}: {nerr(y, y_ref):.3e}"
        # and against the CPU oracle, not only against the library's other entry point
        assert nerr(y, _oracle_y(p, flags)) <= TOL_F32, f"call {seed} vs oracle"


def test_noalloc_forward_frozen_preacts_and_bf16_activations():
    """The frozen-preact forward keeps two tables in the built-in array; bfloat16 activations use the same scratch."""
    from qkan_b200 import _abi

    flags = _abi.QK_FAST_MEASURE | _abi.QK_USE_POSTACT_BIAS
    p = random_problem(61, 96, 48, 24, 3, use_pb=True)
    y, y_ref = _call_both(p, flags)
    assert nerr(y, y_ref) <= TOL_F32 and nerr(y, _oracle_y(p, flags)) <= TOL_F32
    p["x"] = torch.as_tensor(p["x"]).to(torch.bfloat16).float().numpy()
    yb, yb_ref = _call_both(p, flags | _abi.QK_PREACT_TRAINABLE, io_dtype=torch.bfloat16)
    assert nerr(yb, yb_ref) <= TOL_F32
    assert nerr(yb, _oracle_y(p, flags | _abi.QK_PREACT_TRAINABLE)) <= TOL_BF16


def test_noalloc_keeps_its_capacity_for_frozen_preacts():
    """256 x 256 at 3 repetitions with frozen preacts: the two-table form needs 10.5 MB, more than the built-in
    8 MiB, so the entry point runs the one-table form by itself; same results within the float32 bound."""
    from qkan_b200 import _abi

    lib = _abi.load()
    flags = _abi.QK_FAST_MEASURE | _abi.QK_USE_POSTACT_BIAS
    desc = _abi.QkDesc(48, 256, 256, 3, _abi.QK_F32, _abi.QK_F32, flags, 0)
    assert lib.qk_forward_workspace_bytes(_abi.desc_pointer(desc)) > lib.qk_noalloc_max_scratch_bytes()
    p = random_problem(63, 48, 256, 256, 3, use_pb=True)
    y, y_ref = _call_both(p, flags)
    assert nerr(y, y_ref) <= TOL_F32 and nerr(y, _oracle_y(p, flags)) <= TOL_F32


def test_noalloc_forward_on_a_second_device():
    """Each GPU has its own copy of the built-in array and its own looked-up address."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from qkan_b200 import _abi

    flags = _abi.QK_PREACT_TRAINABLE | _abi.QK_FAST_MEASURE | _abi.QK_USE_POSTACT_BIAS
    p = random_problem(62, 80, 40, 24, 2, use_pb=True)
    try:
        for index in (1, 0, 1):
            y, y_ref = _call_both(p, flags, device_index=index)
            assert nerr(y, y_ref) <= TOL_F32, f"device {index}"
    finally:
        torch.cuda.set_device(0)


def test_noalloc_answers_an_unsupported_descriptor_like_the_regular_entry_point():
    from qkan_b200 import _abi

    lib = _abi.load()
    one = torch.zeros(1, device="cuda")
    for desc, want in ((_abi.QkDesc(8, 4, 3, 17, _abi.QK_F32, _abi.QK_F32, 0, 0), _abi.QK_ERR_UNSUPPORTED),
                       (_abi.QkDesc(8, 4, 3, 2, _abi.QK_F32, _abi.QK_F32, 0, 9), _abi.QK_ERR_BAD_ARGUMENT)):
        rc = lib.qk_pz_forward_noalloc(_abi.desc_pointer(desc), *([one.data_ptr()] * 9), None)
        assert rc == want
        assert lib.qk_noalloc_last_error()


def test_noalloc_rejects_problems_beyond_the_built_in_scratch():
    from qkan_b200 import _abi

    lib = _abi.load()
    limit = lib.qk_noalloc_max_scratch_bytes()
    assert limit == 8 << 20
    desc = _abi.QkDesc(4, 2048, 2048, 3, _abi.QK_F32, _abi.QK_F32, _abi.QK_FAST_MEASURE, 0)
    assert lib.qk_forward_workspace_bytes(_abi.desc_pointer(desc)) > limit
    one = torch.zeros(1, device="cuda")
    rc = lib.qk_pz_forward_noalloc(_abi.desc_pointer(desc), *([one.data_ptr()] * 9), None)
    assert rc == _abi.QK_ERR_WORKSPACE
    assert b"scratch" in lib.qk_noalloc_last_error()
