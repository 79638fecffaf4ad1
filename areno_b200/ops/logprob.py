"""Selected-token log-probabilities (and entropy) from logits, vocab-parallel aware.

Forward keeps only four fp32 numbers per row (max, sum-exp, sum-exp·x, target logit); shards
combine through the optional ``tp_group``.  Backward overwrites the saved logits buffer in
place with d(loss)/d(logits), so no probability tensor is ever stored.

Counterpart of ``areno/engine/runtime/logprobs.py:80-235`` in the reference.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib


def selected_logprobs_reference(logits, targets, vocab_start=0, tp_group=None, need_entropy=False):
    x = logits.float()
    m = x.max(-1).values
    if tp_group is not None:
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=tp_group)
    e = torch.exp(x - m[:, None])
    s = e.sum(-1)
    sx = (e * x).sum(-1)
    local = targets - vocab_start
    inside = (local >= 0) & (local < x.shape[-1])
    tgt = torch.where(inside, x.gather(-1, local.clamp(0, x.shape[-1] - 1)[:, None]).squeeze(-1), torch.zeros_like(m))
    if tp_group is not None:
        dist.all_reduce(s, group=tp_group)
        dist.all_reduce(sx, group=tp_group)
        dist.all_reduce(tgt, group=tp_group)
    lse = m + torch.log(s)
    lp = tgt - lse
    if need_entropy:
        return lp, lse - sx / s
    return lp


def _stats(logits, targets, vocab_start):
    rows, v = logits.shape
    dev = logits.device
    out = torch.empty((4, rows), dtype=torch.float32, device=dev)
    _lib.check_index("logprob targets", targets, 1 << 31)
    _lib.call(
        "areno_logprob_stats", logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0), rows, v,
        targets.data_ptr(), vocab_start, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), out[3].data_ptr(),
        _lib.stream(),
    )
    return out


_lib.register_signature("areno_gemm_bf16_lse", "ppiiillplifpppppp" + "p")
_lib.register_signature("areno_gemm_lse_partials_elems", "ii")

_LSE_SCRATCH: dict[int, torch.Tensor] = {}


def fused_head_stats(hidden, weight, targets, vocab_start: int, valid: int, softcap: float = 0.0):
    """Per-row ``(max, sum exp, sum exp x, target logit)`` of ``hidden @ weight[:valid]^T`` computed in the GEMM
    epilogue: the logits are never written.  Returns fp32 ``[4, rows]`` like ``_stats``."""
    rows, k = hidden.shape
    n = weight.shape[0]
    assert hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    if hidden.stride(1) != 1:
        hidden = hidden.contiguous()
    out = torch.empty((4, rows), dtype=torch.float32, device=hidden.device)
    if rows == 0:
        return out
    lib = _lib._load()
    lib.areno_gemm_lse_partials_elems.restype = ctypes.c_longlong
    need = int(lib.areno_gemm_lse_partials_elems(rows, n))
    idx = hidden.device.index if hidden.device.index is not None else torch.cuda.current_device()
    scratch = _LSE_SCRATCH.get(idx)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(need, dtype=torch.float32, device=hidden.device)
        _LSE_SCRATCH[idx] = scratch
    _lib.call("areno_gemm_bf16_lse", hidden.data_ptr(), weight.data_ptr(), rows, n, k, hidden.stride(0), weight.stride(0),
              targets.data_ptr(), int(vocab_start), int(valid), float(softcap or 0.0), scratch.data_ptr(),
              out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), out[3].data_ptr(),
              _lib.status_buffer(hidden.device).data_ptr(), _lib.stream())
    return out


def _combine(stats, tp_group):
    m, s, sx, tgt = stats[0], stats[1], stats[2], stats[3]
    if tp_group is not None and dist.get_world_size(tp_group) > 1:
        gm = m.clone()
        dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=tp_group)
        w = torch.exp(m - gm)
        packed = torch.stack([s * w, sx * w, tgt])
        dist.all_reduce(packed, group=tp_group)
        s, sx, tgt, m = packed[0], packed[1], packed[2], gm
    lse = m + torch.log(s)
    return tgt - lse, lse, sx / s


class _SelectedLogprobs(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, vocab_start, tp_group, need_entropy):
        stats = _stats(logits, targets, vocab_start)
        lp, lse, ex = _combine(stats, tp_group)
        ctx.save_for_backward(logits, targets, lse, ex)
        ctx.vocab_start = vocab_start
        ctx.need_entropy = need_entropy
        if need_entropy:
            return lp, lse - ex
        return lp

    @staticmethod
    def backward(ctx, dlp, dent=None):
        logits, targets, lse, ex = ctx.saved_tensors
        dlp = dlp.float().contiguous()
        if dent is not None:
            dent = dent.float().contiguous()
        # in place: the logits buffer becomes its own gradient
        _lib.call(
            "areno_logprob_bwd", logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0),
            logits.shape[0], logits.shape[1], targets.data_ptr(), ctx.vocab_start, lse.data_ptr(), ex.data_ptr(),
            dlp.data_ptr(), _lib.ptr(dent), _lib.stream(),
        )
        return logits, None, None, None, None


def selected_logprobs(logits, targets, vocab_start: int = 0, tp_group=None, need_entropy: bool = False):
    """log softmax(logits)[target] per row (fp32), optionally with the row entropy.

    logits: ``[rows, V_local]`` bf16 or fp32 (consumed: its storage is reused for the gradient).
    targets: int64 global token ids.
    """
    if targets.dtype != torch.int64:
        targets = targets.to(torch.int64)
    if not logits.is_cuda:
        return selected_logprobs_reference(logits, targets, vocab_start, tp_group, need_entropy)
    assert logits.stride(1) == 1
    targets = targets.contiguous()
    if torch.is_grad_enabled() and logits.requires_grad:
        return _SelectedLogprobs.apply(logits, targets, vocab_start, tp_group, need_entropy)
    lp, lse, ex = _combine(_stats(logits, targets, vocab_start), tp_group)
    if need_entropy:
        return lp, lse - ex
    return lp
