"""bf16 GEMM on the tcgen05 tensor cores and the ``linear`` autograd op built on it.

``gemm`` computes ``D[M,N] = sum_k A(m,k) B(n,k)``.  Each operand may be stored K-major
(``[rows, K]``) or MN-major (``[K, rows]``), which gives forward, dgrad and wgrad of a linear
layer without transposes.  The wgrad can accumulate straight into an fp32 ``main_grad``
buffer in the kernel epilogue.

Counterpart of ``areno/accel/linear.py`` and ``areno/accel/csrc/linear.cu:147-249`` in the
reference (a cuBLAS wrapper there; a hand-written TMA + tcgen05 + TMEM kernel here).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib

EPI_BF16 = 0
EPI_BF16_BIAS = 1
EPI_F32 = 2
EPI_F32_ACC = 3


def _gemm_reference(a, b, a_mn, b_mn, bias, out, accumulate, out_dtype):
    am = a.t() if a_mn else a
    bm = b.t() if b_mn else b
    d = am.float() @ bm.float().t()
    if bias is not None:
        d = d + bias.float()
    if out is not None:
        if accumulate:
            out.add_(d.to(out.dtype))
        else:
            out.copy_(d.to(out.dtype))
        return out
    return d.to(out_dtype)


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    accumulate: bool = False,
    out_dtype: torch.dtype = torch.bfloat16,
    bn: int = 0,
) -> torch.Tensor:
    """``D = A · Bᵀ`` in the logical (row, K) view of both operands.

    a: ``[M, K]`` (or ``[K, M]`` when ``a_mn``), b: ``[N, K]`` (or ``[K, N]`` when ``b_mn``).
    ``out`` may be bf16 or fp32; ``accumulate`` (fp32 only) adds into it.
    """
    if not a.is_cuda:
        return _gemm_reference(a, b, a_mn, b_mn, bias, out, accumulate, out_dtype)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gemm operands must be bf16"
    assert a.dim() == 2 and b.dim() == 2
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    if a_mn:
        k, m = a.shape
    else:
        m, k = a.shape
    if b_mn:
        kb, n = b.shape
    else:
        n, kb = b.shape
    assert k == kb, f"contraction mismatch {k} vs {kb}"
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (m, n) and out.stride(1) == 1
    if out.dtype == torch.bfloat16:
        assert not accumulate, "accumulate requires an fp32 output"
        epi = EPI_BF16_BIAS if bias is not None else EPI_BF16
    else:
        assert out.dtype == torch.float32 and bias is None
        epi = EPI_F32_ACC if accumulate else EPI_F32
    if m == 0 or n == 0:
        return out
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == n
    status = _lib.status_buffer(a.device)
    ws_ptr, ws_bytes = None, 0
    if m <= 512 and epi <= EPI_BF16_BIAS and n <= 18944 and k >= 512 and (m <= 128 or not b_mn):
        # split-K partials of a problem with few output tiles (at most 16 splits; fewer as rows grow)
        ws = _workspace(a.device, 16 * m * n * 4 if m <= 128 else min(8 * m * n * 4, 64 << 20))
        ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
    elif m > 128:
        ws = _workspace(a.device, 0)                      # K slices of the last partial wave (at most 148 tiles)
        ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
    _lib.call(
        "areno_gemm_bf16",
        a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias),
        m, n, k, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn), int(b_mn), epi, bn, ws_ptr, ws_bytes, status.data_ptr(), _lib.stream(),
    )
    return out


_WORKSPACES: dict[int, torch.Tensor] = {}
_RETIRED: list[torch.Tensor] = []     # outgrown workspaces, kept alive for graphs captured while they were current


@dataclass
class SplitKPartial:
    """A skinny GEMM whose split-K partials (fp32 ``[splits, rows, n]``) still sit in the shared
    workspace.  Must be consumed (``ops.norm.splitk_residual_rmsnorm``) before the next GEMM on the
    same device, which reuses that workspace."""

    ws: torch.Tensor
    splits: int
    rows: int
    n: int


def gemm_partials(x: torch.Tensor, weight: torch.Tensor):
    """``x [rows, K] @ weight[N, K]^T`` for decode-sized ``rows``: returns a ``SplitKPartial`` when the
    kernel split K (the fold is left to a fused consumer) or the finished bf16 tensor otherwise."""
    rows, k = x.shape
    n = weight.shape[0]
    if not x.is_contiguous():
        x = x.contiguous()
    out = torch.empty((rows, n), dtype=torch.bfloat16, device=x.device)
    ws = _workspace(x.device, 16 * rows * n * 4)
    splits = ctypes.c_int(1)
    _lib.call("areno_gemm_bf16_partials", x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, n, k, x.stride(0),
              weight.stride(0), n, ws.data_ptr(), ws.numel(), ctypes.byref(splits), _lib.status_buffer(x.device).data_ptr(),
              _lib.stream())
    if splits.value <= 1:
        return out
    return SplitKPartial(ws, int(splits.value), rows, n)


def gated_linear(x: torch.Tensor, weight: torch.Tensor, act: str) -> torch.Tensor:
    """``act(x Wg^T) * (x Wu^T)`` for a merged ``weight = [Wg; Wu]`` (``[2 I, K]``) with the activation in the
    GEMM epilogue; no autograd (inference).  Equal to ``linear`` followed by the gated activation."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and not torch.is_grad_enabled()
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    inter = weight.shape[0] // 2
    out = torch.empty((m, inter), dtype=torch.bfloat16, device=x.device)
    if m == 0:
        return out
    _lib.call("areno_gemm_bf16_gated", x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, inter, k, x.stride(0),
              weight.stride(0), out.stride(0), 0 if act == "silu" else 1, _lib.status_buffer(x.device).data_ptr(),
              _lib.stream())
    return out


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Per-device split-K scratch (uint8), grown on demand and reused by every skinny GEMM.

    Calls on one stream serialise on it; the buffer must not be shared across streams that
    run concurrently.
    """
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _WORKSPACES.get(idx)
    if ws is not None:
        _lib.check_canary("GEMM split-K workspace", ws)      # checked mode: did the previous user stay inside it?
    if ws is None or _usable(ws) < nbytes:
        if ws is not None:
            _RETIRED.append(ws)     # a captured CUDA graph may still point at it: never hand it back to the allocator
        ws = _lib.with_canary(max(nbytes, 32 << 20), torch.device("cuda", idx))
        _WORKSPACES[idx] = ws
    return ws[: _usable(ws)] if _lib.BOUNDS_CHECK else ws


def _usable(ws: torch.Tensor) -> int:
    """Bytes of a workspace in front of its canary (checked mode) or all of it."""
    return ws.numel() - 16 if _lib.BOUNDS_CHECK else ws.numel()


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        y = gemm(x2, weight, bias=bias)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.in_shape = shape
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or (dy2.stride(0) % 8) != 0:
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                # fused fp32 accumulation: main_grad += dyᵀ x, no bf16 grad tensor is materialised
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
                weight.grad_added_to_main_grad = True
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``y = x Wᵀ (+ b)`` with tcgen05 forward, dgrad and wgrad."""
    if not x.is_cuda:
        return torch.nn.functional.linear(x, weight, bias)
    return _Linear.apply(x, weight, bias)
