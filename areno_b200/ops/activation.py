"""Gated and plain activations (SwiGLU, GeGLU-tanh, SiLU, sigmoid, softplus).

Counterpart of ``areno/accel/activations.py`` / ``areno/accel/csrc/activation.cu:18-305``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib

_KIND = {"silu": 0, "gelu_tanh": 1}
_UNARY = {"silu": 0, "sigmoid": 1, "softplus": 2}


def gated_act_reference(x, kind="silu"):
    g, u = x.float().chunk(2, dim=-1)
    a = F.silu(g) if kind == "silu" else F.gelu(g, approximate="tanh")
    return (a * u).to(x.dtype)


class _GatedAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kind):
        I = x.shape[-1] // 2
        x2 = x.reshape(-1, 2 * I)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        out = torch.empty((x2.shape[0], I), dtype=x.dtype, device=x.device)
        _lib.call("areno_gated_act_fwd", x2.data_ptr(), out.data_ptr(), x2.shape[0], I, kind, _lib.stream())
        ctx.save_for_backward(x2)
        ctx.kind = kind
        ctx.shape = x.shape
        return out.view(*x.shape[:-1], I)

    @staticmethod
    def backward(ctx, dout):
        (x2,) = ctx.saved_tensors
        I = x2.shape[-1] // 2
        d2 = dout.reshape(-1, I)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dx = torch.empty_like(x2)
        _lib.call("areno_gated_act_bwd", d2.data_ptr(), x2.data_ptr(), dx.data_ptr(), x2.shape[0], I, ctx.kind,
                  _lib.stream())
        return dx.view(ctx.shape), None


_lib.register_signature("areno_gated_act_fwd_rows", "ppplii" + "p")


def _gated_rows(x, kind: int, row_route):
    """Inference on an expert-sorted buffer: only rows with a route are computed, the rest stays unspecified."""
    I = x.shape[-1] // 2
    x2 = x.contiguous()
    out = torch.empty((x2.shape[0], I), dtype=x.dtype, device=x.device)
    _lib.call("areno_gated_act_fwd_rows", x2.data_ptr(), out.data_ptr(), row_route.data_ptr(), x2.shape[0], I, kind,
              _lib.stream())
    return out


def silu_and_mul(x, row_route=None):
    """``silu(x[..., :I]) * x[..., I:]``.  ``row_route`` (int32 per row, negative = padding) restricts the work to
    the routed rows of an expert-sorted buffer; only honoured when no gradient is needed."""
    if not x.is_cuda:
        return gated_act_reference(x, "silu")
    if row_route is not None and x.dim() == 2 and not torch.is_grad_enabled():
        return _gated_rows(x, 0, row_route)
    return _GatedAct.apply(x, 0)


def gelu_tanh_and_mul(x, row_route=None):
    """``gelu_tanh(x[..., :I]) * x[..., I:]`` (``row_route``: see ``silu_and_mul``)."""
    if not x.is_cuda:
        return gated_act_reference(x, "gelu_tanh")
    if row_route is not None and x.dim() == 2 and not torch.is_grad_enabled():
        return _gated_rows(x, 1, row_route)
    return _GatedAct.apply(x, 1)


class _Unary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kind):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _lib.call("areno_unary_act", xc.data_ptr(), None, y.data_ptr(), xc.numel(), kind, 0, _lib.stream())
        ctx.save_for_backward(xc)
        ctx.kind = kind
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        _lib.call("areno_unary_act", xc.data_ptr(), dyc.data_ptr(), dx.data_ptr(), xc.numel(), ctx.kind, 1,
                  _lib.stream())
        return dx, None


def _unary(x, name):
    if not x.is_cuda or x.dtype != torch.bfloat16:
        xf = x.float()
        if name == "silu":
            return F.silu(xf).to(x.dtype)
        if name == "sigmoid":
            return torch.sigmoid(xf).to(x.dtype)
        return F.softplus(xf, threshold=20.0).to(x.dtype)
    return _Unary.apply(x, _UNARY[name])


def silu(x):
    return _unary(x, "silu")


def sigmoid(x):
    return _unary(x, "sigmoid")


def softplus(x):
    return _unary(x, "softplus")
