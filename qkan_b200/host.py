"""Forward + backward of one layer for callers whose activations live in host memory.

The reference keeps everything in torch tensors and leaves host/device movement to the
user (``QKAN.train_`` simply calls ``.to(self.device)`` per batch, ``src/qkan/qkan.py:1794-1795``).
For batches that arrive in (pinned) host memory this helper hides the PCIe transfers behind the
kernels: the batch is cut into row chunks, and three streams run as a pipeline —

    copy-in   : x, grad_y of chunk k+1   host -> device
    compute   : forward, backward of chunk k   (the C-ABI kernels)
    copy-out  : y, grad_x of chunk k-1   device -> host

Rows are independent, so chunking changes nothing but the order in which the batch-summed
parameter gradients are accumulated (chunk partial sums are added in chunk order: still
run-to-run reproducible).

Chunk boundaries sit on multiples of ``row_align`` rows (default: 148 SMs x 64 rows, one full wave of
forward tiles and, at 256 columns, of backward tiles), so that cutting the batch does not add partly
filled waves of CTAs. Successive steps overlap too: the copy-out of one step's last chunk runs under the
next step's first kernels (``wait()`` orders the current stream after everything queued so far).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import functional as qf
from .parallel import GradBucket, layer_grad_shapes


def chunk_spans(batch: int, n_chunks: int, row_align: int = 148 * 64):
    """Row ranges ``[(begin, end), ...]`` of at most ``n_chunks`` chunks covering ``batch`` rows.

    The chunk length is rounded up to a multiple of ``row_align`` (whole waves of CTAs) when the batch holds
    at least two such units; the last chunk takes the remainder.
    """
    if batch <= 0:
        return []
    n_chunks = max(1, min(n_chunks, batch))
    step = (batch + n_chunks - 1) // n_chunks
    if row_align > 1 and batch >= 2 * row_align:
        step = (step + row_align - 1) // row_align * row_align
    return [(b, min(batch, b + step)) for b in range(0, batch, step)]


class HostLayerPipeline:
    """Chunked, stream-overlapped ``y, grad_x, parameter gradients`` from host-resident ``x, grad_y``."""

    #: library launches of one step(): 1 set-up + (forward + backward + finish) per chunk
    def launches_per_step(self) -> int:
        return 1 + 3 * len(self.spans)

    def __init__(self, batch: int, in_dim: int, out_dim: int, reps: int, device, *, n_chunks: int = 3,
                 dtype: torch.dtype = torch.float32, preact_trainable: bool = True,
                 fast_measure: bool = True, use_postact_bias: bool = True, ansatz: str = "pz_encoding",
                 row_align: int = 148 * 64):
        self.device = torch.device(device)
        self.cfg = dict(preact_trainable=preact_trainable, fast_measure=fast_measure,
                        use_postact_bias=use_postact_bias, ansatz=ansatz)
        self.spans = chunk_spans(batch, n_chunks, row_align)
        dev = self.device
        self.dx = [torch.empty((e - b, in_dim), dtype=dtype, device=dev) for b, e in self.spans]
        self.dgy = [torch.empty((e - b, out_dim), dtype=dtype, device=dev) for b, e in self.spans]
        self.dgx = [torch.empty((e - b, in_dim), dtype=dtype, device=dev) for b, e in self.spans]
        self.dy = [torch.empty((e - b, out_dim), dtype=dtype, device=dev) for b, e in self.spans]
        shapes = layer_grad_shapes(in_dim, out_dim, reps, preact_trainable=preact_trainable,
                                   postact_bias=use_postact_bias)
        if ansatz in ("rpz_encoding", "rpz"):
            shapes["theta"] = (out_dim, in_dim, reps + 1, 1)
        elif ansatz == "real":
            shapes["theta"] = (out_dim, in_dim, reps, 1)
        self.bucket = GradBucket(shapes, dev)                      # the summed gradients
        self.chunk_buckets = [GradBucket(shapes, dev) for _ in self.spans]
        self.s_in = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        self.ev_in = [torch.cuda.Event() for _ in self.spans]
        self.ev_done = [torch.cuda.Event() for _ in self.spans]
        self.ev_free = [torch.cuda.Event() for _ in self.spans]    # chunk buffers drained by copy-out
        self.ev_sum = torch.cuda.Event()                            # summed gradients ready
        self.ev_sum_free = torch.cuda.Event()                       # ... and copied out
        self._first = True

    def step(self, hx: torch.Tensor, hgy: torch.Tensor, params: Dict[str, Optional[torch.Tensor]],
             hy: torch.Tensor, hgx: torch.Tensor, hgrads: Optional[torch.Tensor] = None) -> GradBucket:
        """Queue one forward+backward. ``hx, hgy, hy, hgx, hgrads`` are pinned host tensors; ``params`` holds the
        device tensors theta, pw, pb, postw, postb (basew / mask optional). Returns the gradient bucket
        (device; valid for work queued on the current stream). Host results are complete after ``wait()`` plus a
        synchronisation of the current stream, or after ``torch.cuda.synchronize()``."""
        compute = torch.cuda.current_stream(self.device)
        p = params
        # the per-edge tables are built once per step and serve every chunk (they have no batch axis)
        prep = qf.prepare_layer(p["theta"], p["pw"], p["pb"], p["postw"], p.get("postb"), p.get("basew"),
                                p.get("mask"), in_dim=self.dx[0].shape[1], **self.cfg)
        for k, (b, e) in enumerate(self.spans):
            with torch.cuda.stream(self.s_in):
                if not self._first:
                    self.s_in.wait_event(self.ev_free[k])  # previous step finished reading this chunk's buffers
                self.dx[k].copy_(hx[b:e], non_blocking=True)
                self.dgy[k].copy_(hgy[b:e], non_blocking=True)
                self.ev_in[k].record(self.s_in)
            compute.wait_event(self.ev_in[k])
            if not self._first:
                compute.wait_event(self.ev_free[k])  # the previous step's y and grad_x of this chunk have left the device
            y = qf.forward_prepared(prep, self.dx[k], out=self.dy[k])
            outs = dict(self.chunk_buckets[k].views, x=self.dgx[k])
            qf.backward_prepared(prep, self.dx[k], self.dgy[k], out=outs, want=tuple(outs))
            self.ev_done[k].record(compute)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_done[k])
                hy[b:e].copy_(y, non_blocking=True)
                hgx[b:e].copy_(self.dgx[k], non_blocking=True)
                self.ev_free[k].record(self.s_out)
        flat = self.bucket.flat
        if not self._first:
            compute.wait_event(self.ev_sum_free)  # the previous step's gradients have left the device
        self._first = False
        flat.copy_(self.chunk_buckets[0].flat)
        for cb in self.chunk_buckets[1:]:
            flat.add_(cb.flat)
        self.bucket.all_reduce()
        self.ev_sum.record(compute)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_sum)
            if hgrads is not None:
                hgrads.copy_(flat, non_blocking=True)
            self.ev_sum_free.record(self.s_out)
        return self.bucket

    def wait(self) -> None:
        """Order the current stream after every copy queued so far (host results are then one stream sync away)."""
        torch.cuda.current_stream(self.device).wait_stream(self.s_out)
