"""Tensor-level entry points over the C ABI: the fused layer op and the solver-contract op.

``qkan_layer`` is the body of the reference's ``QKANLayer._forward_train`` after the
optional batch-norm (``src/qkan/qkan.py:755-785``) as one differentiable op;
``qkan_postacts`` is the reference's solver contract (``src/qkan/solver/_base.py:29-51``).
torch is used for device memory, the current stream and autograd bookkeeping only.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _abi


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch owned by the caller side of the ABI: a fresh block from torch's caching allocator per call.

    The allocator hands the same cached block back call after call (no ``cudaMalloc`` once warm), keeps blocks
    apart per stream, and inside a CUDA-graph capture takes them from the graph's private pool, so a captured
    address can never be handed to anyone else. 512-byte alignment is the allocator's own.
    """
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _io_dtype(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _abi.QK_F32
    if t.dtype == torch.bfloat16:
        return _abi.QK_BF16
    raise TypeError(f"qkan_b200 computes on float32 or bfloat16 activations, got {t.dtype}")


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"qkan_b200: `{name}` is on {t.device}; the B200 kernels are the only compute path "
            "(no CPU fallback)")


def _f32c(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.float32).contiguous()


def _flags(preact_trainable: bool, fast_measure: bool, use_postact_bias: bool, precise: bool = False) -> int:
    return ((_abi.QK_PREACT_TRAINABLE if preact_trainable else 0)
            | (_abi.QK_FAST_MEASURE if fast_measure else 0)
            | (_abi.QK_USE_POSTACT_BIAS if use_postact_bias else 0)
            | (_abi.QK_PRECISE_MATH if precise else 0))


# Layers up to this many edge evaluations per call default to the full-precision math path when
# `precise="auto"`: they cost microseconds either way, and small fits are where LBFGS needs smooth gradients.
AUTO_PRECISE_MAX_EDGES = 1 << 22


def resolve_precise(precise, x: torch.Tensor, out_dim: int) -> bool:
    """Turn True / False / "auto" into the flag: auto = float32 activations and a small layer."""
    if precise == "auto" or precise is None:
        return x.dtype == torch.float32 and x.shape[0] * x.shape[1] * out_dim <= AUTO_PRECISE_MAX_EDGES
    return bool(precise)


def _oi_params(postw, postb, basew, mask):
    """Bring the (O,I) tensors to one dtype (float32 or bfloat16) and contiguity."""
    tensors = [t for t in (postw, postb, basew, mask) if t is not None]
    dt = torch.bfloat16 if all(t.dtype == torch.bfloat16 for t in tensors) else torch.float32
    conv = lambda t: None if t is None else t.detach().to(dt).contiguous()  # noqa: E731
    return conv(postw), conv(postb), conv(basew), conv(mask), (_abi.QK_BF16 if dt == torch.bfloat16 else _abi.QK_F32)


def _ansatz_code(ansatz) -> int:
    try:
        return _abi.ANSATZ_CODES[ansatz]
    except (KeyError, TypeError):
        raise NotImplementedError(
            f"ansatz {ansatz!r}: the B200 kernels implement pz_encoding, rpz_encoding and real") from None


def _make_desc(x, theta, flags, param_dtype, ansatz="pz_encoding", out_dim: Optional[int] = None) -> _abi.QkDesc:
    """Descriptor from the tensor shapes.

    Per-edge theta is (O,I,R+1,2) pz, (O,I,R+1,1) rpz, (O,I,R,1) real. Grouped theta drops the (O,I) axes
    for one group axis, ``(g, ...)``: edge (o,i) uses entry ``i mod g`` (``src/qkan/solver/exact.py:68-86``);
    the number of outputs then comes from ``out_dim``.
    """
    code = _ansatz_code(ansatz)
    B, I = x.shape
    width_want = 2 if code == _abi.QK_ANSATZ_PZ else 1
    if theta.dim() == 3:
        group, layers, width = theta.shape
        if out_dim is None or group < 1:
            raise ValueError("grouped theta (3 dimensions) needs out_dim and at least one group entry")
        O = int(out_dim)
    elif theta.dim() == 4:
        O, I2, layers, width = theta.shape
        group = 0
        if I2 != I or (out_dim is not None and out_dim != O):
            raise ValueError(f"theta {tuple(theta.shape)} does not match x {tuple(x.shape)} / out_dim {out_dim}")
    else:
        raise ValueError(f"theta must have 4 dimensions (3 when grouped), got {tuple(theta.shape)}")
    if width != width_want:
        raise ValueError(f"theta {tuple(theta.shape)} does not match ansatz {ansatz!r}")
    reps = layers if code == _abi.QK_ANSATZ_REAL else layers - 1
    return _abi.QkDesc(B, I, O, reps, _io_dtype(x), param_dtype, flags, code, group)


def _preact_shape(desc: _abi.QkDesc):
    return (desc.group, desc.reps) if desc.group else (desc.out_dim, desc.in_dim, desc.reps)


class PreparedLayer:
    """Per-edge constants of one layer for unchanged parameters: the output of ``qk_pz_prepare``.

    ``tables`` is the device buffer the ``*_prepared`` entry points read; ``postw`` / ``postb`` / ``mask`` are the
    converted (O,I) tensors the backward's finishing kernel reads again. The state has no batch axis: it serves
    any number of rows, float32 or bfloat16 activations, until a parameter value changes.
    """

    __slots__ = ("tables", "postw", "postb", "mask", "has_base", "shape", "reps", "flags", "param_dtype",
                 "ansatz_code", "group", "theta_shape")

    def desc(self, x: torch.Tensor) -> _abi.QkDesc:
        if x.dim() != 2 or x.shape[1] != self.shape[1]:
            raise ValueError(f"x {tuple(x.shape)} does not match the prepared layer ({self.shape[1]} inputs)")
        return _abi.QkDesc(x.shape[0], self.shape[1], self.shape[0], self.reps, _io_dtype(x), self.param_dtype,
                           self.flags, self.ansatz_code, self.group)


def prepare_layer(theta, pw, pb, postw, postb=None, basew=None, mask=None, *, in_dim: int,
                  preact_trainable: bool, fast_measure: bool = True, use_postact_bias: bool = False,
                  ansatz: str = "pz_encoding", precise: bool = False) -> PreparedLayer:
    """Run the set-up kernel once (``qk_pz_prepare``): tables and folded bias for these parameter values."""
    lib = _abi.load()
    _require_cuda(theta, "theta")
    dev = theta.device
    theta, pw, pb = _f32c(theta), _f32c(pw), _f32c(pb)
    postw, postb, basew, mask, pdt = _oi_params(postw, postb if use_postact_bias else None, basew, mask)
    flags = _flags(preact_trainable, fast_measure, use_postact_bias and postb is not None, precise)
    probe = torch.empty((0, in_dim), dtype=torch.float32, device="meta")
    d = _make_desc(probe, theta, flags, pdt, ansatz, out_dim=postw.shape[0])
    prep = PreparedLayer()
    prep.postw, prep.postb, prep.mask, prep.has_base = postw, postb, mask, basew is not None
    prep.shape, prep.reps, prep.flags, prep.param_dtype = (d.out_dim, d.in_dim), d.reps, flags, pdt
    prep.ansatz_code, prep.group, prep.theta_shape = d.ansatz, d.group, tuple(theta.shape)
    with torch.cuda.device(dev):
        nbytes = lib.qk_tables_bytes(_abi.desc_pointer(d))
        _abi.check(0 if nbytes else _abi.QK_ERR_BAD_ARGUMENT, "qk_tables_bytes")
        prep.tables = _workspace(dev, nbytes)
        rc = lib.qk_pz_prepare(_abi.desc_pointer(d), _ptr(theta), _ptr(pw), _ptr(pb), _ptr(postw), _ptr(postb),
                               _ptr(basew), _ptr(mask), _ptr(prep.tables), prep.tables.numel(),
                               torch.cuda.current_stream(dev).cuda_stream)
    _abi.check(rc, "qk_pz_prepare")
    return prep


def _check_out(t, shape, dtype, dev, name):
    if (tuple(t.shape) != tuple(shape) and t.numel() != torch.Size(shape).numel()) or t.dtype != dtype \
            or t.device != dev or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous {dtype} tensor of {tuple(shape)} on {dev}")


def forward_prepared(prep: PreparedLayer, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y (B,O)`` from prepared tables: one launch (``qk_pz_forward_prepared``)."""
    lib = _abi.load()
    _require_cuda(x, "x")
    x = x.detach().contiguous()
    desc = prep.desc(x)
    if out is None:
        y = torch.empty((x.shape[0], desc.out_dim), dtype=x.dtype, device=x.device)
    else:
        y = out
        if tuple(y.shape) != (x.shape[0], desc.out_dim):
            raise ValueError(f"out must be a contiguous {x.dtype} tensor of {(x.shape[0], desc.out_dim)} on {x.device}")
        _check_out(y, (x.shape[0], desc.out_dim), x.dtype, x.device, "out")
    with torch.cuda.device(x.device):
        rc = lib.qk_pz_forward_prepared(_abi.desc_pointer(desc), _ptr(x), _ptr(prep.tables), prep.tables.numel(),
                                        int(prep.has_base), _ptr(y), torch.cuda.current_stream(x.device).cuda_stream)
    _abi.check(rc, "qk_pz_forward_prepared")
    return y


_GRAD_NAMES = ("x", "theta", "preacts_weight", "preacts_bias", "postact_weights", "postact_bias", "base_weight")


def backward_prepared(prep: PreparedLayer, x: torch.Tensor, gy: torch.Tensor, *, want=_GRAD_NAMES,
                      out: Optional[dict] = None) -> dict:
    """Gradients from prepared tables: backward + finish launches (``qk_pz_backward_prepared``)."""
    lib = _abi.load()
    _require_cuda(x, "x")
    x = x.detach().contiguous()
    gy = gy.detach().to(x.dtype).contiguous()
    desc = prep.desc(x)
    O, I = desc.out_dim, desc.in_dim
    dev = x.device
    shapes = {"x": tuple(x.shape), "theta": prep.theta_shape, "preacts_weight": _preact_shape(desc),
              "preacts_bias": _preact_shape(desc), "postact_weights": (O, I), "postact_bias": (O, I),
              "base_weight": (O, I)}
    given = out or {}
    out = {}
    for name in want:
        dt = x.dtype if name == "x" else torch.float32
        t = given.get(name)
        if t is None:
            t = torch.empty(shapes[name], dtype=dt, device=dev)
        else:
            _check_out(t, shapes[name], dt, dev, f"out[{name!r}]")
        out[name] = t
    with torch.cuda.device(dev):
        nbytes = lib.qk_backward_scratch_bytes(_abi.desc_pointer(desc))
        ws = _workspace(dev, nbytes)
        rc = lib.qk_pz_backward_prepared(
            _abi.desc_pointer(desc), _ptr(x), _ptr(prep.tables), prep.tables.numel(), _ptr(prep.postw),
            _ptr(prep.postb), _ptr(prep.mask), int(prep.has_base), _ptr(gy), _ptr(out.get("x")),
            _ptr(out.get("theta")), _ptr(out.get("preacts_weight")), _ptr(out.get("preacts_bias")),
            _ptr(out.get("postact_weights")), _ptr(out.get("postact_bias")), _ptr(out.get("base_weight")),
            _ptr(ws), ws.numel(), torch.cuda.current_stream(dev).cuda_stream)
    _abi.check(rc, "qk_pz_backward_prepared")
    return out


def edge_stats(prep: PreparedLayer, x: torch.Tensor) -> torch.Tensor:
    """Unbiased standard deviation over the batch of every edge's output, ``(O,I)`` float32 (``qk_pz_edge_stats``).

    Equal to ``torch.std(forward_no_sum(x), dim=0)`` of the reference (``src/qkan/qkan.py:835-891, 1287-1292``)
    without the ``(B,O,I)`` tensor; no autograd (the reference computes it under ``no_grad`` as well).
    """
    lib = _abi.load()
    _require_cuda(x, "x")
    x = x.detach().contiguous()
    desc = prep.desc(x)
    out = torch.empty((desc.out_dim, desc.in_dim), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        nbytes = lib.qk_edge_stats_scratch_bytes(_abi.desc_pointer(desc))
        ws = _workspace(x.device, nbytes)
        rc = lib.qk_pz_edge_stats(_abi.desc_pointer(desc), _ptr(x), _ptr(prep.tables), prep.tables.numel(),
                                  int(prep.has_base), _ptr(out), _ptr(ws), ws.numel(),
                                  torch.cuda.current_stream(x.device).cuda_stream)
    _abi.check(rc, "qk_pz_edge_stats")
    return out


def layer_forward(x, theta, pw, pb, postw, postb=None, basew=None, mask=None, *,
                  preact_trainable: bool, fast_measure: bool = True,
                  use_postact_bias: bool = False, ansatz: str = "pz_encoding",
                  precise: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y (B,O)`` of the fused layer; no autograd (see ``qkan_layer``). ``out``: preallocated contiguous result.

    Set-up and forward in one C-ABI call (``qk_pz_forward``); with unchanged parameters use ``prepare_layer`` once
    and ``forward_prepared`` / ``backward_prepared`` after it.
    """
    lib = _abi.load()
    _require_cuda(x, "x")
    x = x.detach().contiguous()
    theta, pw, pb = _f32c(theta), _f32c(pw), _f32c(pb)
    postw, postb, basew, mask, pdt = _oi_params(postw, postb if use_postact_bias else None, basew, mask)
    desc = _make_desc(x, theta, _flags(preact_trainable, fast_measure, use_postact_bias and postb is not None, precise), pdt, ansatz,
                      out_dim=postw.shape[0])
    if out is None:
        y = torch.empty((x.shape[0], desc.out_dim), dtype=x.dtype, device=x.device)
    else:
        y = out
        if (tuple(y.shape) != (x.shape[0], desc.out_dim) or y.dtype != x.dtype or y.device != x.device
                or not y.is_contiguous()):
            raise ValueError(f"out must be a contiguous {x.dtype} tensor of {(x.shape[0], desc.out_dim)} on {x.device}")
    with torch.cuda.device(x.device):
        nbytes = lib.qk_forward_workspace_bytes(_abi.desc_pointer(desc))
        ws = _workspace(x.device, nbytes)
        rc = lib.qk_pz_forward(_abi.desc_pointer(desc), _ptr(x), _ptr(theta), _ptr(pw), _ptr(pb),
                               _ptr(postw), _ptr(postb), _ptr(basew), _ptr(mask), _ptr(y),
                               _ptr(ws), ws.numel(), torch.cuda.current_stream(x.device).cuda_stream)
    _abi.check(rc, "qk_pz_forward")
    return y


def layer_backward(x, theta, pw, pb, postw, postb, basew, mask, gy, *, preact_trainable: bool,
                   fast_measure: bool = True, use_postact_bias: bool = False,
                   want=_GRAD_NAMES, out: Optional[dict] = None,
                   ansatz: str = "pz_encoding", precise: bool = False) -> dict:
    """Gradients of ``sum(y * gy)`` named as the reference's parameters; float32 except ``x``.

    ``out`` may hold preallocated contiguous destination tensors by name (for example the views
    of a ``parallel.GradBucket``); the kernels overwrite them, they do not accumulate.
    """
    lib = _abi.load()
    _require_cuda(x, "x")
    x = x.detach().contiguous()
    gy = gy.detach().to(x.dtype).contiguous()
    theta, pw, pb = _f32c(theta), _f32c(pw), _f32c(pb)
    postw, postb, basew, mask, pdt = _oi_params(postw, postb if use_postact_bias else None, basew, mask)
    desc = _make_desc(x, theta, _flags(preact_trainable, fast_measure, use_postact_bias and postb is not None, precise), pdt, ansatz,
                      out_dim=postw.shape[0])
    O, I = desc.out_dim, desc.in_dim
    dev = x.device
    shapes = {"x": tuple(x.shape), "theta": tuple(theta.shape), "preacts_weight": _preact_shape(desc),
              "preacts_bias": _preact_shape(desc), "postact_weights": (O, I), "postact_bias": (O, I),
              "base_weight": (O, I)}
    given = out or {}
    out = {}
    for name in want:
        dt = x.dtype if name == "x" else torch.float32
        t = given.get(name)
        if t is None:
            t = torch.empty(shapes[name], dtype=dt, device=dev)
        elif (t.dtype != dt or t.device != dev or not t.is_contiguous()
              or t.numel() != torch.Size(shapes[name]).numel()):
            raise ValueError(f"out[{name!r}] must be a contiguous {dt} tensor of {shapes[name]} on {dev}")
        out[name] = t
    with torch.cuda.device(dev):
        nbytes = lib.qk_backward_workspace_bytes(_abi.desc_pointer(desc))
        ws = _workspace(dev, nbytes)
        rc = lib.qk_pz_backward(
            _abi.desc_pointer(desc), _ptr(x), _ptr(theta), _ptr(pw), _ptr(pb), _ptr(postw),
            _ptr(postb), _ptr(basew), _ptr(mask), _ptr(gy), _ptr(out.get("x")),
            _ptr(out.get("theta")), _ptr(out.get("preacts_weight")), _ptr(out.get("preacts_bias")),
            _ptr(out.get("postact_weights")), _ptr(out.get("postact_bias")),
            _ptr(out.get("base_weight")), _ptr(ws), ws.numel(),
            torch.cuda.current_stream(dev).cuda_stream)
    _abi.check(rc, "qk_pz_backward")
    return out


def postacts_forward(x, theta, pw, pb, *, preact_trainable: bool, fast_measure: bool = True,
                     ansatz: str = "pz_encoding", precise: bool = False,
                     out_dim: Optional[int] = None) -> torch.Tensor:
    """Per-edge activations ``(B,O,I)`` (solver contract); no autograd. ``out_dim`` is needed for grouped theta."""
    lib = _abi.load()
    _require_cuda(x, "x")
    x = x.detach().contiguous()
    theta, pw, pb = _f32c(theta), _f32c(pw), _f32c(pb)
    desc = _make_desc(x, theta, _flags(preact_trainable, fast_measure, False, precise), _abi.QK_F32, ansatz, out_dim)
    out = torch.empty((x.shape[0], desc.out_dim, x.shape[1]), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        nbytes = lib.qk_forward_workspace_bytes(_abi.desc_pointer(desc))
        ws = _workspace(x.device, nbytes)
        rc = lib.qk_pz_postacts_forward(_abi.desc_pointer(desc), _ptr(x), _ptr(theta), _ptr(pw),
                                        _ptr(pb), _ptr(out), _ptr(ws), ws.numel(),
                                        torch.cuda.current_stream(x.device).cuda_stream)
    _abi.check(rc, "qk_pz_postacts_forward")
    return out


def postacts_backward(x, theta, pw, pb, gpostacts, *, preact_trainable: bool,
                      fast_measure: bool = True,
                      want=("x", "theta", "preacts_weight", "preacts_bias"),
                      ansatz: str = "pz_encoding", precise: bool = False,
                      out_dim: Optional[int] = None) -> dict:
    lib = _abi.load()
    _require_cuda(x, "x")
    x = x.detach().contiguous()
    gpostacts = gpostacts.detach().to(x.dtype).contiguous()
    theta, pw, pb = _f32c(theta), _f32c(pw), _f32c(pb)
    desc = _make_desc(x, theta, _flags(preact_trainable, fast_measure, False, precise), _abi.QK_F32, ansatz, out_dim)
    f32 = dict(dtype=torch.float32, device=x.device)
    out = {}
    if "x" in want:
        out["x"] = torch.empty_like(x)
    if "theta" in want:
        out["theta"] = torch.empty(tuple(theta.shape), **f32)
    if "preacts_weight" in want:
        out["preacts_weight"] = torch.empty(_preact_shape(desc), **f32)
    if "preacts_bias" in want:
        out["preacts_bias"] = torch.empty(_preact_shape(desc), **f32)
    with torch.cuda.device(x.device):
        nbytes = lib.qk_backward_workspace_bytes(_abi.desc_pointer(desc))
        ws = _workspace(x.device, nbytes)
        rc = lib.qk_pz_postacts_backward(
            _abi.desc_pointer(desc), _ptr(x), _ptr(theta), _ptr(pw), _ptr(pb), _ptr(gpostacts),
            _ptr(out.get("x")), _ptr(out.get("theta")), _ptr(out.get("preacts_weight")),
            _ptr(out.get("preacts_bias")), _ptr(ws), ws.numel(),
            torch.cuda.current_stream(x.device).cuda_stream)
    _abi.check(rc, "qk_pz_postacts_backward")
    return out


def _uses_preacts(preact_trainable: bool, ansatz: str) -> bool:
    """rpz always encodes pw*x + pb, so its preact gradients exist whatever the flag says."""
    return preact_trainable or _ansatz_code(ansatz) == _abi.QK_ANSATZ_RPZ


class _LayerFunction(torch.autograd.Function):
    """Forward: set-up + forward kernel; the prepared tables are kept for the backward (two more launches)."""

    @staticmethod
    def forward(ctx, x, theta, pw, pb, postw, postb, basew, mask, preact_trainable, fast_measure,
                use_postact_bias, ansatz, precise):
        prep = prepare_layer(theta, pw, pb, postw, postb, basew, mask, in_dim=x.shape[1],
                             preact_trainable=preact_trainable, fast_measure=fast_measure,
                             use_postact_bias=use_postact_bias, ansatz=ansatz, precise=precise)
        y = forward_prepared(prep, x)
        ctx.save_for_backward(x)
        ctx.prep = prep
        ctx.cfg = (preact_trainable, use_postact_bias, ansatz)
        ctx.meta = [(t.dtype, t.shape) if t is not None else None for t in (x, theta, pw, pb, postw, postb, basew)]
        return y

    @staticmethod
    def backward(ctx, gy):
        (x,) = ctx.saved_tensors
        prep = ctx.prep
        preact_trainable, use_postact_bias, ansatz = ctx.cfg
        need = ctx.needs_input_grad
        want = tuple(n for k, n in enumerate(_GRAD_NAMES) if need[k])
        if not _uses_preacts(preact_trainable, ansatz):
            want = tuple(n for n in want if n not in ("preacts_weight", "preacts_bias"))
        if prep.postb is None or not use_postact_bias:
            want = tuple(n for n in want if n != "postact_bias")
        if not prep.has_base:
            want = tuple(n for n in want if n != "base_weight")
        g = backward_prepared(prep, x, gy, want=want)
        outs = []
        for k, n in enumerate(_GRAD_NAMES):
            t = g.get(n)
            if t is not None and ctx.meta[k] is not None:
                dtype, shape = ctx.meta[k]
                t = t.to(dtype).reshape(shape)
            outs.append(t)
        return (*outs, None, None, None, None, None, None)


def qkan_layer(x, theta, preacts_weight, preacts_bias, postact_weights, postact_bias=None,
               base_weight=None, mask=None, *, preact_trainable: bool, fast_measure: bool = True,
               use_postact_bias: bool = False, ansatz: str = "pz_encoding", precise="auto") -> torch.Tensor:
    """Differentiable fused QKAN layer ``(B,I) -> (B,O)`` on the CUDA kernels.

    ``precise``: True / False / "auto" (see ``resolve_precise``) selects full-precision sin/cos/sqrt
    instead of the special-function unit.
    """
    return _LayerFunction.apply(x, theta, preacts_weight, preacts_bias, postact_weights,
                                postact_bias, base_weight, mask, preact_trainable, fast_measure,
                                use_postact_bias, ansatz, resolve_precise(precise, x, postact_weights.shape[0]))


class _PostactsFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, theta, pw, pb, preact_trainable, fast_measure, ansatz, precise, out_dim):
        ctx.save_for_backward(x, theta, pw, pb)
        ctx.cfg = (preact_trainable, fast_measure, ansatz, precise, out_dim)
        return postacts_forward(x, theta, pw, pb, preact_trainable=preact_trainable,
                                fast_measure=fast_measure, ansatz=ansatz, precise=precise, out_dim=out_dim)

    @staticmethod
    def backward(ctx, gpa):
        x, theta, pw, pb = ctx.saved_tensors
        preact_trainable, fast_measure, ansatz, precise, out_dim = ctx.cfg
        names = ("x", "theta", "preacts_weight", "preacts_bias")
        need = ctx.needs_input_grad
        want = tuple(n for k, n in enumerate(names) if need[k])
        if not _uses_preacts(preact_trainable, ansatz):
            want = tuple(n for n in want if n not in ("preacts_weight", "preacts_bias"))
        g = postacts_backward(x, theta, pw, pb, gpa, preact_trainable=preact_trainable,
                              fast_measure=fast_measure, want=want, ansatz=ansatz, precise=precise,
                              out_dim=out_dim)
        srcs = (x, theta, pw, pb)
        outs = []
        for k, n in enumerate(names):
            t = g.get(n)
            if t is not None:
                t = t.to(srcs[k].dtype).reshape(srcs[k].shape)
            outs.append(t)
        return (*outs, None, None, None, None, None)


def qkan_postacts(x, theta, preacts_weight, preacts_bias, *, preact_trainable: bool,
                  fast_measure: bool = True, ansatz: str = "pz_encoding", precise="auto",
                  out_dim: Optional[int] = None) -> torch.Tensor:
    """Differentiable per-edge activations ``(B,O,I)`` — the reference solver contract.

    Grouped theta / preacts ``(g, ...)`` are read in place (pass ``out_dim``); their gradients come back grouped."""
    O = theta.shape[0] if theta.dim() == 4 else out_dim
    return _PostactsFunction.apply(x, theta, preacts_weight, preacts_bias, preact_trainable,
                                   fast_measure, ansatz, resolve_precise(precise, x, O), out_dim)
