"""Two CPU ranks over gloo: the gradient bucket all-reduce and the row sharding used by the N-GPU path."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qkan_b200.parallel import GradBucket, OverlappedGradSync, layer_grad_shapes, shard_rows, sync_module_grads


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      LOCAL_RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bucket = GradBucket(layer_grad_shapes(4, 3, 2), "cpu")
        # each rank's "gradient" is a function of its row shard: the sum must equal the full-batch value
        rows = torch.arange(10, dtype=torch.float32)
        b, e = shard_rows(10, rank, world)
        for k, name in enumerate(bucket.names):
            bucket[name].fill_(float(rows[b:e].sum()) * (k + 1))
        bucket.all_reduce()
        ok = all(torch.allclose(bucket[name], torch.full_like(bucket[name], 45.0 * (k + 1)))
                 for k, name in enumerate(bucket.names))
        lin = torch.nn.Linear(3, 2)
        for p in lin.parameters():
            p.grad = torch.full_like(p, float(rank + 1))
        moved = sync_module_grads(lin, average=True)
        ok = ok and all(torch.allclose(p.grad, torch.full_like(p, 1.5)) for p in lin.parameters())
        ok = ok and moved == 4 * sum(p.numel() for p in lin.parameters())
        out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_bucket_allreduce_world_size_2():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]


def _spawn(target, world=2, timeout=180):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=timeout) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return results


def _lbfgs_worker(rank: int, world: int, port: int, out):
    """train_ with LBFGS + strong-Wolfe line search on different row shards: every rank must issue the same
    collectives (no hang) and end with identical parameters."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      LOCAL_RANK=str(rank), WORLD_SIZE=str(world))
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        from qkan_b200 import QKAN

        torch.manual_seed(0)
        # width [3, 1] with the map head: no circuit layer, so the loop runs on CPU tensors; the training loop,
        # its closure and its collectives are the ones every model uses
        model = QKAN([3, 1], is_map=True, hidden=8, device="cpu", seed=0)
        gen = torch.Generator().manual_seed(100 + rank)  # each rank sees its own rows
        xs = torch.rand(64, 3, generator=gen)
        ys = torch.sin(3 * xs.sum(dim=1, keepdim=True)) + 0.3 * rank
        data = {"train_input": xs, "train_label": ys, "test_input": xs[:16], "test_label": ys[:16]}
        opt = torch.optim.LBFGS(model.parameters(), lr=0.5, line_search_fn="strong_wolfe", max_iter=6,
                                tolerance_change=1e-7)
        sched = torch.optim.lr_scheduler.ReduceLROnPlateau(opt, patience=0, factor=0.5)
        res = model.train_(data, optimizer=opt, scheduler=sched, steps=4, verbose=False)
        flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
        gathered = [torch.zeros_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        same = all(torch.equal(gathered[0], g) for g in gathered)
        losses = torch.tensor([float(v) for v in res["train_loss"]])
        lg = [torch.zeros_like(losses) for _ in range(world)]
        dist.all_gather(lg, losses)
        same = same and all(torch.equal(lg[0], g) for g in lg)
        out.put((rank, bool(same), opt.param_groups[0]["lr"]))
    finally:
        dist.destroy_process_group()


def test_train_lbfgs_strong_wolfe_world_size_2_stays_in_step():
    results = _spawn(_lbfgs_worker)
    assert [r[:2] for r in results] == [(0, True), (1, True)]
    assert results[0][2] == results[1][2]  # the plateau scheduler took the same decisions on both ranks


def _overlap_worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      LOCAL_RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Tanh(), torch.nn.Linear(7, 3), torch.nn.Tanh(),
                                    torch.nn.Linear(3, 1))
        full_x = torch.rand(12, 5, generator=torch.Generator().manual_seed(5))
        full_t = torch.rand(12, 1, generator=torch.Generator().manual_seed(6))
        # whole-batch gradients, computed locally, are the expected averaged shard gradients
        torch.nn.functional.mse_loss(model(full_x), full_t).backward()
        want = [p.grad.clone() for p in model.parameters()]
        model.zero_grad(set_to_none=True)
        merged = OverlappedGradSync(model)  # small layers share a bucket
        ok = len(merged.groups) == 1
        merged.remove()
        sync = OverlappedGradSync(model, min_bucket_bytes=0)
        ok = ok and len(sync.groups) == 3
        b, e = shard_rows(12, rank, world)
        for _ in range(2):  # twice: the buckets are cleared and re-armed by zero_grad()
            sync.zero_grad()
            torch.nn.functional.mse_loss(model(full_x[b:e]), full_t[b:e]).backward()
            sync.finish()
            ok = ok and all(torch.allclose(p.grad, w, atol=1e-6) for p, w in zip(model.parameters(), want))
        out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_overlapped_layer_buckets_world_size_2():
    assert _spawn(_overlap_worker) == [(0, True), (1, True)]
