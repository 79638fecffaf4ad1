"""RMSNorm family: plain, fused residual-add, optional-scale, Gemma-style (1 + w) offset.

CUDA tensors run the sm_100a kernels of ``csrc/elementwise.cu``; CPU tensors run the fp32
PyTorch restatement below, which is also the numerical oracle of the tests.
Counterpart of ``areno/accel/normalization.py`` / ``areno/accel/csrc/normalization.cu:33-264``.
"""

from __future__ import annotations

import torch

from . import _lib


def rmsnorm_reference(x, weight, eps, residual=None, w_offset=0.0):
    h = x.float()
    if residual is not None:
        h = (h + residual.float()).to(x.dtype).float()
    inv = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    y = h * inv
    if weight is not None:
        y = y * (weight.float() + w_offset)
    y = y.to(x.dtype)
    if residual is not None:
        return y, h.to(x.dtype)
    return y


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, eps, w_offset):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        inv = torch.empty(rows, dtype=torch.float32, device=x.device)
        h_out = None
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, H)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            h_out = torch.empty_like(x2)
        wf32 = int(weight is not None and weight.dtype == torch.float32)
        _lib.call(
            "areno_rmsnorm_fwd",
            x2.data_ptr(), _lib.ptr(r2), _lib.ptr(weight), wf32, float(w_offset),
            y.data_ptr(), _lib.ptr(h_out), inv.data_ptr(), rows, H, float(eps), _lib.stream(),
        )
        h_saved = h_out if h_out is not None else x2
        ctx.save_for_backward(h_saved, weight, inv)
        ctx.w_offset = w_offset
        ctx.shape = x.shape
        ctx.has_res = residual is not None
        ctx.has_w = weight is not None
        ctx.mark_non_differentiable()
        if residual is not None:
            return y.view(x.shape), h_out.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        h, weight, inv = ctx.saved_tensors
        H = h.shape[-1]
        rows = h.shape[0]
        dy2 = dy.reshape(-1, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if dh is not None:
            dres = dh.reshape(-1, H)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(h)
        dw = None
        partial = None
        dw_target = None
        accumulate = 0
        if ctx.has_w and ctx.needs_input_grad[1]:
            nblk = _lib.fn("areno_rmsnorm_bwd_blocks")(rows)
            partial = torch.empty((nblk, H), dtype=torch.float32, device=h.device)
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                dw_target = main_grad
                accumulate = 1
                weight.grad_added_to_main_grad = True
            else:
                dw_target = torch.empty(H, dtype=torch.float32, device=h.device)
        wf32 = int(weight is not None and weight.dtype == torch.float32)
        _lib.call(
            "areno_rmsnorm_bwd",
            dy2.data_ptr(), h.data_ptr(), _lib.ptr(weight), wf32, float(ctx.w_offset), inv.data_ptr(),
            _lib.ptr(dres), dx.data_ptr(), _lib.ptr(partial), _lib.ptr(dw_target), accumulate, rows, H,
            _lib.stream(),
        )
        if dw_target is not None and not accumulate:
            dw = dw_target.to(weight.dtype)
        dxv = dx.view(ctx.shape)
        return dxv, dw, (dxv if ctx.has_res else None), None, None


def splitk_residual_rmsnorm(part, residual, weight, eps: float = 1e-6, w_offset: float = 0.0):
    """Fold the split-K partials of a skinny GEMM, add the residual stream and apply RMSNorm in one
    kernel (inference only).  Returns ``(y, h)`` with ``h = residual + sum of partials``."""
    rows, n = part.rows, part.n
    dev = part.ws.device
    h = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
    y = torch.empty_like(h)
    if residual is not None and not residual.is_contiguous():
        residual = residual.contiguous()
    _lib.call("areno_splitk_residual_rmsnorm", part.ws.data_ptr(), part.splits, rows * n, _lib.ptr(residual),
              weight.data_ptr(), int(weight.dtype == torch.float32), float(w_offset), y.data_ptr(), h.data_ptr(), rows, n,
              float(eps), _lib.stream())
    return y, h


def rmsnorm(x, weight, eps: float = 1e-6, residual=None, w_offset: float = 0.0):
    """``y = h · rsqrt(mean h² + eps) · (w + w_offset)`` with ``h = x (+ residual)``.

    With ``residual`` the call returns ``(y, h)`` so the caller keeps the updated residual
    stream without a separate add kernel.  ``weight=None`` gives the scale-free norm.
    """
    if not x.is_cuda:
        return rmsnorm_reference(x, weight, eps, residual, w_offset)
    return _RMSNorm.apply(x, weight, residual, eps, w_offset)
