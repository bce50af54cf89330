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

_WORKSPACES: dict = {}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch owned by the caller side of the ABI: one growing buffer per (device, stream)."""
    stream = torch.cuda.current_stream(device)
    key = (device.index, stream.cuda_stream)
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buf
    return buf


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


def layer_forward(x, theta, pw, pb, postw, postb=None, basew=None, mask=None, *,
                  preact_trainable: bool, fast_measure: bool = True,
                  use_postact_bias: bool = False, ansatz: str = "pz_encoding",
                  precise: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y (B,O)`` of the fused layer; no autograd (see ``qkan_layer``). ``out``: preallocated contiguous result."""
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
                   want=("x", "theta", "preacts_weight", "preacts_bias", "postact_weights",
                         "postact_bias", "base_weight"), out: Optional[dict] = None,
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
    @staticmethod
    def forward(ctx, x, theta, pw, pb, postw, postb, basew, mask, preact_trainable, fast_measure,
                use_postact_bias, ansatz, precise):
        # theta / preacts reach the kernels as float32; converted once here and kept for the backward
        theta32, pw32, pb32 = _f32c(theta), _f32c(pw), _f32c(pb)
        ctx.save_for_backward(x, theta32, pw32, pb32, postw, postb, basew, mask)
        ctx.cfg = (preact_trainable, fast_measure, use_postact_bias, ansatz, precise)
        ctx.meta = [(t.dtype, t.shape) if t is not None else None for t in (x, theta, pw, pb, postw, postb, basew)]
        return layer_forward(x, theta32, pw32, pb32, postw, postb, basew, mask,
                             preact_trainable=preact_trainable, fast_measure=fast_measure,
                             use_postact_bias=use_postact_bias, ansatz=ansatz, precise=precise)

    @staticmethod
    def backward(ctx, gy):
        x, theta, pw, pb, postw, postb, basew, mask = ctx.saved_tensors
        preact_trainable, fast_measure, use_postact_bias, ansatz, precise = ctx.cfg
        names = ("x", "theta", "preacts_weight", "preacts_bias", "postact_weights", "postact_bias",
                 "base_weight")
        need = ctx.needs_input_grad
        want = tuple(n for k, n in enumerate(names) if need[k])
        if not _uses_preacts(preact_trainable, ansatz):
            want = tuple(n for n in want if n not in ("preacts_weight", "preacts_bias"))
        if postb is None or not use_postact_bias:
            want = tuple(n for n in want if n != "postact_bias")
        if basew is None:
            want = tuple(n for n in want if n != "base_weight")
        g = layer_backward(x, theta, pw, pb, postw, postb, basew, mask, gy,
                           preact_trainable=preact_trainable, fast_measure=fast_measure,
                           use_postact_bias=use_postact_bias, want=want, ansatz=ansatz, precise=precise)
        outs = []
        for k, n in enumerate(names):
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
