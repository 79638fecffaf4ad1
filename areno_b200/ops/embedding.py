"""Vocab-parallel embedding lookup.

Rows whose id falls outside ``[vocab_start, vocab_end)`` produce zeros (another rank owns
them).  The backward scatter-adds in fp32, directly into ``weight.main_grad`` when present.
Counterpart of ``areno/accel/embedding.py`` / ``areno/accel/csrc/embedding.cu:10-104``.
"""

from __future__ import annotations

import torch

from . import _lib


def embedding_reference(ids, table, vocab_start=0, scale=1.0):
    v1 = vocab_start + table.shape[0]
    mask = (ids >= vocab_start) & (ids < v1)
    local = (ids - vocab_start).clamp(0, table.shape[0] - 1)
    out = torch.nn.functional.embedding(local, table)
    out = out * mask.unsqueeze(-1).to(out.dtype)
    if scale != 1.0:
        out = (out.float() * scale).to(table.dtype)
    return out


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, vocab_start, scale):
        flat = ids.reshape(-1)
        if flat.dtype != torch.int64:
            flat = flat.to(torch.int64)
        flat = flat.contiguous()
        H = table.shape[1]
        _lib.check_index("embedding ids", flat, 1 << 31)      # negative ids are never valid; the shard test covers the rest
        out = torch.empty((flat.numel(), H), dtype=table.dtype, device=table.device)
        _lib.call("areno_embedding_fwd", flat.data_ptr(), table.data_ptr(), out.data_ptr(), flat.numel(), H,
                  vocab_start, vocab_start + table.shape[0], float(scale), _lib.stream())
        ctx.save_for_backward(flat)
        ctx.table = table
        ctx.args = (vocab_start, scale)
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):
        (flat,) = ctx.saved_tensors
        table = ctx.table
        vocab_start, scale = ctx.args
        H = table.shape[1]
        d2 = dout.reshape(-1, H)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        main_grad = getattr(table, "main_grad", None)
        if main_grad is not None:
            target = main_grad
            table.grad_added_to_main_grad = True
        else:
            target = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        _lib.call("areno_embedding_bwd", flat.data_ptr(), d2.data_ptr(), target.data_ptr(), flat.numel(), H,
                  vocab_start, vocab_start + table.shape[0], float(scale), _lib.stream())
        dw = None if main_grad is not None else target.to(table.dtype)
        return None, dw, None, None


def embedding(ids, table, vocab_start: int = 0, scale: float = 1.0, out: torch.Tensor | None = None):
    """``out`` (inference only, CUDA): write the rows into this contiguous ``[ids.numel(), H]`` tensor."""
    if not table.is_cuda:
        res = embedding_reference(ids, table, vocab_start, scale)
        return res if out is None else out.copy_(res)
    if out is not None:
        flat = ids.reshape(-1)
        if flat.dtype != torch.int64:
            flat = flat.to(torch.int64)
        flat = flat.contiguous()
        assert out.is_contiguous() and out.shape == (flat.numel(), table.shape[1]) and out.dtype == table.dtype
        _lib.check_index("embedding ids", flat, 1 << 31)
        _lib.call("areno_embedding_fwd", flat.data_ptr(), table.data_ptr(), out.data_ptr(), flat.numel(), table.shape[1],
                  vocab_start, vocab_start + table.shape[0], float(scale), _lib.stream())
        return out
    return _Embedding.apply(ids, table, vocab_start, scale)
