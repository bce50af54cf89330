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


def mean_over_ranks(value: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """The mean of a scalar over the ranks (detached); the value itself without an initialised process group.

    A training loop must hand its optimiser and its scheduler the SAME number on every rank: LBFGS decides from
    the loss how many more closure calls (each one a collective) to make, and a plateau scheduler decides from
    it when to cut the learning rate. Per-rank losses would let the ranks drift apart, or deadlock.
    """
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return value
    out = value.detach().clone().to(torch.float32)
    dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
    return (out / dist.get_world_size(group)).to(value.dtype)


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


class OverlappedGradSync:
    """Data-parallel gradient averaging for a multi-layer model, one collective per layer, overlapped with backward.

    The parameters are grouped layer by layer (``groups``: by default each direct child of ``module.layers``, or
    of ``module`` itself). Each group's ``.grad`` tensors are views of one flat float32 buffer. Autograd
    accumulates into the views; a post-accumulate hook counts the group's parameters as they become ready, and
    when the last one is, the group's buffer is all-reduced asynchronously on the collective stream while autograd
    goes on with the layers nearer the input. ``finish()`` waits for the collectives and applies the 1/world
    average. The reference has no counterpart (it leaves data parallelism to the user, ``src/qkan/info.py:62-75``);
    the rows of a batch are independent, so this sum is the only exchange of a training step.

    Usage per step: ``sync.zero_grad(); loss.backward(); sync.finish(); optimizer.step()``. Do not call
    ``optimizer.zero_grad(set_to_none=True)`` in between: it would detach the views (``zero_grad()`` here
    re-attaches them).
    """

    def __init__(self, module: torch.nn.Module, groups: Optional[list] = None,
                 group: Optional[dist.ProcessGroup] = None, average: bool = True,
                 min_bucket_bytes: int = 1 << 20):
        if groups is None:
            children = list(getattr(module, "layers", module).children()) or [module]
            groups = [[p for p in c.parameters() if p.requires_grad] for c in children]
            seen = {id(p) for g in groups for p in g}
            rest = [p for p in module.parameters() if p.requires_grad and id(p) not in seen]
            if rest:
                groups.append(rest)
        # neighbouring layers whose gradients are small share a bucket: below about a megabyte a collective is all
        # latency, and one launch for two layers beats two
        merged: list = []
        for g in (g for g in groups if g):
            if merged and sum(p.numel() for p in merged[-1]) * 4 < min_bucket_bytes:
                merged[-1] = merged[-1] + list(g)
            else:
                merged.append(list(g))
        self.groups = merged
        self.pg, self.average = group, average
        # NCCL averages inside the collective; other backends (gloo in the CPU tests) sum, and finish() divides
        self._avg_in_collective = False
        if average and dist.is_available() and dist.is_initialized():
            self._avg_in_collective = dist.get_backend(group) == "nccl"
        self.flats, self._pending, self._handles, self._hooks = [], [], [], []
        for gi, params in enumerate(self.groups):
            dev = params[0].device
            n = sum((p.numel() + 63) // 64 * 64 for p in params)
            flat = torch.zeros(n, dtype=torch.float32, device=dev)
            self.flats.append(flat)
            self._pending.append(0)
            for p in params:
                if p.dtype != torch.float32:
                    raise TypeError("OverlappedGradSync buckets float32 parameters; keep low-precision copies outside")
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(gi)))
        self._attach()

    def _attach(self) -> None:
        for flat, params in zip(self.flats, self.groups):
            off = 0
            for p in params:
                p.grad = flat[off: off + p.numel()].view_as(p)
                off += (p.numel() + 63) // 64 * 64

    def _make_hook(self, gi: int):
        def hook(_param):
            self._pending[gi] -= 1
            if self._pending[gi] == 0:
                self._launch(gi)
        return hook

    def _launch(self, gi: int) -> None:
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.pg) > 1:
            op = dist.ReduceOp.AVG if self._avg_in_collective else dist.ReduceOp.SUM
            self._handles.append(dist.all_reduce(self.flats[gi], op=op, group=self.pg, async_op=True))

    def zero_grad(self) -> None:
        """Clear the buckets, re-attach the views and arm the ready counters for the next backward."""
        for gi, flat in enumerate(self.flats):
            flat.zero_()
            self._pending[gi] = len(self.groups[gi])
        self._handles = []
        self._attach()

    def finish(self) -> None:
        """Wait for the collectives of this backward (groups whose hooks never fired, because a parameter
        got no gradient, are reduced here) and turn the sums into means."""
        for gi, left in enumerate(self._pending):
            if left > 0:
                self._pending[gi] = 0
                self._launch(gi)
        for h in self._handles:
            h.wait()
        self._handles = []
        if self.average and not self._avg_in_collective and dist.is_available() and dist.is_initialized():
            world = dist.get_world_size(self.pg)
            if world > 1:
                for flat in self.flats:
                    flat.div_(world)

    def nbytes(self) -> int:
        return sum(f.numel() * 4 for f in self.flats)

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
