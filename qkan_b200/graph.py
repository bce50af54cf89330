"""CUDA-graph capture of whole-model inference and of one training step.

Small layers are bound by launches rather than by arithmetic: a forward + backward of one QKAN
layer is seven launches of this library plus the autograd bookkeeping around them. The reference
offers the same two helpers for that regime (``src/qkan/inference.py:68-135, 205-330``); here
they are thin wrappers over ``torch.cuda.CUDAGraph``, which works because the kernels launch on
the current stream, never synchronise and take all their memory from the caller.
"""
from __future__ import annotations

from typing import Callable

import torch
from torch import nn


def _warm(fn: Callable[[], None], warmup: int) -> None:
    """Run ``fn`` a few times on a side stream (allocations, lazy initialisation) before capture."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(warmup, 1)):
            fn()
    torch.cuda.current_stream().wait_stream(side)


def make_graphed_inference(model: nn.Module, sample_input: torch.Tensor,
                           warmup: int = 3) -> Callable[[torch.Tensor], torch.Tensor]:
    """Capture ``model(sample_input)`` under ``no_grad``; the returned callable replays it for same-shaped inputs.

    The result is a view of a static buffer that the next call overwrites: clone it to keep it.
    """
    static_x = sample_input.detach().clone()
    with torch.no_grad():
        _warm(lambda: model(static_x), warmup)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_y = model(static_x)

    def replay(x: torch.Tensor) -> torch.Tensor:
        if x.shape != static_x.shape or x.dtype != static_x.dtype:
            raise ValueError(f"graph was captured for {tuple(static_x.shape)} {static_x.dtype}, "
                             f"got {tuple(x.shape)} {x.dtype}")
        static_x.copy_(x)
        graph.replay()
        return static_y

    return replay


def make_graphed_train_step(model: nn.Module, sample_input: torch.Tensor, sample_target: torch.Tensor,
                            loss_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                            optimizer: torch.optim.Optimizer,
                            warmup: int = 3, flat_grads: bool = False) -> Callable[[torch.Tensor, torch.Tensor], torch.Tensor]:
    """Capture forward + loss + gradients; ``optimizer.step()`` stays with the caller.

    After ``loss = step(x, y)`` every trainable parameter's ``.grad`` holds this step's gradient
    (static buffers, overwritten by the next call) and ``loss`` is a static scalar tensor.

    ``flat_grads=True`` gathers the gradients, inside the graph, into one flat float32 buffer (``step.flat``) of
    which the ``.grad`` tensors are views: a data-parallel loop then needs a single all-reduce of ``step.flat``
    between ``step(x, y)`` and ``optimizer.step()``. Parameters without a gradient get zeros.
    """
    static_x = sample_input.detach().clone()
    static_t = sample_target.detach().clone()
    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    params = [p for _, p in named]

    # The step is differentiated with respect to fresh leaf tensors that alias the parameters' storage
    # (so optimizer updates stay visible to the replays), through torch.autograd.grad. Differentiating the
    # parameters themselves would reuse their gradient-accumulation nodes, which stay tied to the stream of
    # an earlier eager step for as long as any old autograd graph is alive, and running those inside a
    # capture on another stream is an error (the reference re-allocates every parameter for this reason,
    # src/qkan/inference.py:137-203).
    def loss_and_grads():
        leaves = {n: p.detach().requires_grad_(True) for n, p in named}
        loss = loss_fn(torch.func.functional_call(model, leaves, (static_x,)), static_t)
        return loss, torch.autograd.grad(loss, list(leaves.values()), allow_unused=True)

    def loss_and_flat():
        loss, grads = loss_and_grads()
        pieces = [(g if g is not None else torch.zeros_like(p)).reshape(-1).to(torch.float32)
                  for g, p in zip(grads, params)]
        return loss, torch.cat(pieces)

    flat = None
    if flat_grads:
        _warm(loss_and_flat, warmup)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_loss, flat = loss_and_flat()
        static_grads, off = [], 0
        for p in params:
            static_grads.append(flat[off: off + p.numel()].view_as(p))
            off += p.numel()
    else:
        _warm(loss_and_grads, warmup)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_loss, static_grads = loss_and_grads()

    def train_step(x: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        if x.shape != static_x.shape or target.shape != static_t.shape:
            raise ValueError("graph was captured for other input / target shapes")
        static_x.copy_(x)
        static_t.copy_(target)
        graph.replay()
        for p, g in zip(params, static_grads):  # re-attach: an optimizer.zero_grad() in between is harmless
            p.grad = g if g is None or g.dtype == p.dtype else g.to(p.dtype)
        return static_loss

    train_step.flat = flat
    return train_step
