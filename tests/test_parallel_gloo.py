"""Two CPU ranks over gloo: the gradient bucket all-reduce and the row sharding used by the N-GPU path."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qkan_b200.parallel import GradBucket, layer_grad_shapes, shard_rows, sync_module_grads


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
