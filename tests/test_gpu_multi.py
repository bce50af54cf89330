"""Two GPUs over NCCL: row-sharded forward/backward + one gradient all-reduce == the single-GPU full batch.

Needs two visible CUDA devices; on a one-GPU box the test is skipped (the bucket logic itself is
covered on CPU ranks in test_parallel_gloo.py).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.util import nerr, random_problem

pytestmark = pytest.mark.gpu

B, I, O, R = 600, 70, 40, 3
CFG = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      LOCAL_RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from qkan_b200 import functional as F
        from qkan_b200.parallel import GradBucket, layer_grad_shapes, shard_rows

        p = random_problem(21, B, I, O, R, use_pb=True)
        b, e = shard_rows(B, rank, world)
        t = {k: torch.from_numpy(v).to(dev) for k, v in p.items() if v is not None}
        x, gy = t["x"][b:e].contiguous(), t["gy"][b:e].contiguous()
        bucket = GradBucket(layer_grad_shapes(I, O, R), dev)
        y = F.layer_forward(x, t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], None, None, **CFG)
        g = F.layer_backward(x, t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], None, None, gy,
                             out=dict(bucket.views), want=tuple(bucket.views) + ("x",), **CFG)
        bucket.all_reduce()
        torch.cuda.synchronize()
        out.put((rank, y.cpu().numpy(), g["x"].cpu().numpy(), {k: v.cpu().numpy() for k, v in bucket.views.items()}))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_data_parallel_matches_single_gpu():
    from qkan_b200 import functional as F

    p = random_problem(21, B, I, O, R, use_pb=True)
    t = {k: torch.from_numpy(v).cuda() for k, v in p.items() if v is not None}
    y_ref = F.layer_forward(t["x"], t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], None, None, **CFG)
    g_ref = F.layer_backward(t["x"], t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], None, None,
                             t["gy"], **CFG)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for pr in procs:
        pr.start()
    results = sorted((out.get(timeout=180) for _ in procs), key=lambda r: r[0])
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    y = np.concatenate([r[1] for r in results])
    gx = np.concatenate([r[2] for r in results])
    assert nerr(y, y_ref.cpu().numpy()) <= 1e-6
    assert nerr(gx, g_ref["x"].cpu().numpy()) <= 1e-6
    for rank_result in results:  # every rank ends with the same, full-batch parameter gradients
        for k, v in rank_result[3].items():
            assert nerr(v, g_ref[k].cpu().numpy()) <= 2e-6, k


def _model_worker(rank: int, world: int, port: int, out):
    """Two-layer model, per-layer gradient buckets reduced under the backward (NCCL, averaged in the collective)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      LOCAL_RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from qkan_b200 import QKAN
        from qkan_b200.parallel import OverlappedGradSync, shard_rows

        model = QKAN([24, 16, 5], reps=2, device=dev, seed=3, preact_trainable=True, ba_trainable=True)
        sync = OverlappedGradSync(model, min_bucket_bytes=0)
        g = torch.Generator().manual_seed(11)
        x = torch.rand(128, 24, generator=g).to(dev)
        t = torch.rand(128, 5, generator=g).to(dev)
        b, e = shard_rows(128, rank, world)
        for _ in range(2):  # the second pass reuses cleared, re-armed buckets
            sync.zero_grad()
            torch.nn.functional.mse_loss(model(x[b:e]), t[b:e]).backward()
            sync.finish()
        torch.cuda.synchronize()
        out.put((rank, len(sync.groups), {n: p.grad.cpu().numpy() for n, p in model.named_parameters()
                                          if p.grad is not None}))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_overlapped_layer_buckets_match_single_gpu():
    from qkan_b200 import QKAN

    model = QKAN([24, 16, 5], reps=2, device="cuda", seed=3, preact_trainable=True, ba_trainable=True)
    g = torch.Generator().manual_seed(11)
    x = torch.rand(128, 24, generator=g).cuda()
    t = torch.rand(128, 5, generator=g).cuda()
    torch.nn.functional.mse_loss(model(x), t).backward()
    want = {n: p.grad.cpu().numpy() for n, p in model.named_parameters() if p.grad is not None}
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_model_worker, args=(r, 2, port, out)) for r in range(2)]
    for pr in procs:
        pr.start()
    results = sorted((out.get(timeout=180) for _ in procs), key=lambda r: r[0])
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    for _, n_groups, grads in results:
        assert n_groups == 2
        assert sorted(grads) == sorted(want)
        for k, v in grads.items():  # equal shards: the mean of the shard means is the full-batch mean
            assert nerr(v, want[k]) <= 5e-6, k
