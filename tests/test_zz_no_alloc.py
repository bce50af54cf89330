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

from tests.util import TOL_F32, nerr, random_problem

pytestmark = pytest.mark.gpu


def _call_both(p, cfg_flags):
    from qkan_b200 import _abi

    lib = _abi.load()
    dev = torch.device("cuda", 0)
    t = {k: (None if v is None else torch.from_numpy(v).to(dev)) for k, v in p.items()}
    B, I = p["x"].shape
    O, _, R1, _ = p["theta"].shape
    desc = _abi.QkDesc(B, I, O, R1 - 1, _abi.QK_F32, _abi.QK_F32, cfg_flags, 0)
    dp = _abi.desc_pointer(desc)
    ptr = lambda k: None if t[k] is None else t[k].data_ptr()  # noqa: E731
    stream = torch.cuda.current_stream(dev).cuda_stream
    # existing entry point with a caller-owned workspace
    nbytes = lib.qk_forward_workspace_bytes(dp)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    y_ref = torch.empty((B, O), device=dev)
    rc = lib.qk_pz_forward(dp, ptr("x"), ptr("theta"), ptr("pw"), ptr("pb"), ptr("postw"), ptr("postb"),
                           ptr("basew"), ptr("mask"), y_ref.data_ptr(), ws.data_ptr(), nbytes, stream)
    assert rc == 0, _abi.last_error()
    # new entry point: no workspace argument at all
    y = torch.empty((B, O), device=dev)
    rc = lib.qk_pz_forward_noalloc(dp, ptr("x"), ptr("theta"), ptr("pw"), ptr("pb"), ptr("postw"),
                                   ptr("postb"), ptr("basew"), ptr("mask"), y.data_ptr(), stream)
    assert rc == 0, lib.qk_noalloc_last_error().decode()
    torch.cuda.synchronize()
    return y.cpu().numpy(), y_ref.cpu().numpy()


def test_noalloc_forward_matches_workspace_forward_twice_in_a_row():
    from qkan_b200 import _abi

    flags = _abi.QK_PREACT_TRAINABLE | _abi.QK_FAST_MEASURE | _abi.QK_USE_POSTACT_BIAS
    # two calls in a row with different shapes and values: the second sees the first one's leftovers
    for seed, (B, I, O, R) in enumerate([(130, 70, 40, 3), (64, 33, 90, 2)]):
        p = random_problem(50 + seed, B, I, O, R, use_pb=True, base=(seed == 1), masked=True)
        y, y_ref = _call_both(p, flags)
        assert np.isfinite(y).all()
        assert nerr(y, y_ref) <= TOL_F32, f"call {seed}: {nerr(y, y_ref):.3e}"


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
