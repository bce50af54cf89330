"""Batch data-parallel plumbing: one process per GPU, replicated parameters, sharded rows.

The reference has no data-parallel code of its own (it only parses ``RANK`` /
``LOCAL_RANK`` / ``WORLD_SIZE``, ``src/qkan/info.py:62-75``, and leaves DDP to the
user). Rows of ``x`` are independent, so the only exchange of a step is one
sum-all-reduce of the parameter gradients. ``GradBucket`` lays the gradient tensors
of a layer out as views of one flat float32 buffer so that the backward writes
straight into it and a single collective (NCCL over NVLink on GPUs, gloo in the CPU
tests) covers all of them.
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, Optional, Tuple

import torch
import torch.distributed as dist


def get_dist_info() -> Tuple[bool, int, int, int]:
    """``(is_distributed, rank, local_rank, world_size)`` from the launcher's environment.

    Same contract as the reference's helper (``src/qkan/info.py:62-75``).
    """
    if int(os.environ.get("RANK", -1)) == -1:
        return False, 0, 0, 1
    for var in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        if var not in os.environ:
            raise RuntimeError(f"{var} is not set although RANK is")
    return True, int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])


def print0(*args, **kwargs) -> None:
    """Print on rank 0 only (``src/qkan/info.py:33-36``)."""
    if int(os.environ.get("RANK", 0)) == 0:
        print(*args, **kwargs)


def shard_rows(n_rows: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous ``[begin, end)`` row range of ``rank``; the first ``n_rows % world_size`` ranks get one extra row."""
    base, extra = divmod(n_rows, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class GradBucket:
    """Gradient tensors as views of one flat float32 buffer, reduced with one collective."""

    def __init__(self, shapes: Dict[str, Iterable[int]], device, dtype=torch.float32):
        self.names = list(shapes)
        self.shapes = {k: tuple(int(s) for s in v) for k, v in shapes.items()}
        sizes = {k: int(torch.Size(v).numel()) for k, v in self.shapes.items()}
        # 64-element (256-byte) alignment of every view keeps vector accesses legal
        self.offsets = {}
        off = 0
        for k in self.names:
            self.offsets[k] = off
            off += (sizes[k] + 63) // 64 * 64
        self.flat = torch.zeros(max(off, 1), dtype=dtype, device=device)
        self.views = {k: self.flat[self.offsets[k]: self.offsets[k] + sizes[k]].view(self.shapes[k])
                      for k in self.names}

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.views[name]

    def all_reduce(self, group: Optional[dist.ProcessGroup] = None, average: bool = False) -> None:
        """Sum (or mean) the bucket over the ranks; a no-op without an initialised process group."""
        if not (dist.is_available() and dist.is_initialized()):
            return
        world = dist.get_world_size(group)
        if world == 1:
            return
        dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            self.flat.div_(world)

    def nbytes(self) -> int:
        return self.flat.numel() * self.flat.element_size()


def bind_host_thread_near_gpu(device_index: int) -> Optional[int]:
    """Pin the calling thread to the CPU cores NVML lists as local to this GPU (same NUMA node / PCIe root).

    With one process per GPU, pinned host buffers allocated afterwards land in memory next to the GPU, so the
    ranks' host<->device copies do not all cross the same inter-socket link. Touches only this process's CPU
    affinity (no GPU setting). Returns the number of cores in the new mask, or None when NVML, the device or
    the container's cpuset does not allow it (nothing is changed then).
    """
    try:
        import pynvml

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        try:
            handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        n_words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, n_words)
        local = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        allowed = local & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return len(allowed)
    except Exception:
        return None


def layer_grad_shapes(in_dim: int, out_dim: int, reps: int, *, preact_trainable: bool = True,
                      postact_bias: bool = True, base: bool = False) -> Dict[str, Tuple[int, ...]]:
    """Shapes of the parameter gradients of one layer, in the order they are packed."""
    shapes: Dict[str, Tuple[int, ...]] = {"theta": (out_dim, in_dim, reps + 1, 2)}
    if preact_trainable:
        shapes["preacts_weight"] = (out_dim, in_dim, reps)
        shapes["preacts_bias"] = (out_dim, in_dim, reps)
    shapes["postact_weights"] = (out_dim, in_dim)
    if postact_bias:
        shapes["postact_bias"] = (out_dim, in_dim)
    if base:
        shapes["base_weight"] = (out_dim, in_dim)
    return shapes


def sync_module_grads(module: torch.nn.Module, group: Optional[dist.ProcessGroup] = None,
                      average: bool = True) -> int:
    """All-reduce every ``.grad`` of ``module`` through one flat buffer; returns the bytes moved.

    Used by the data-parallel training loop for whole models (several layers, plus any
    ordinary torch modules around them).
    """
    grads = [p.grad for p in module.parameters() if p.grad is not None]
    if not grads or not (dist.is_available() and dist.is_initialized()):
        return 0
    world = dist.get_world_size(group)
    if world == 1:
        return 0
    flat = torch.cat([g.reshape(-1).to(torch.float32) for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat.div_(world)
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off: off + n].view_as(g))
        off += n
    return flat.numel() * 4
