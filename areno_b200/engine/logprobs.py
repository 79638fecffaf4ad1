"""LM head fused with selected-token log-prob / entropy, chunked over rows.

Forward: per chunk of rows, logits = hidden · Wᵀ (tcgen05 GEMM), reduced at once to four fp32
numbers per row; the ``[rows, vocab]`` logits are dropped, or kept in bf16 for backward when the
device has room.  Backward: logits are recomputed per chunk (or taken from forward), overwritten in place by their gradient, and fed to the dgrad / wgrad GEMMs (the wgrad
accumulates straight into ``weight.main_grad`` when present).  With a vocab-parallel head the
per-row statistics are combined over the TP group and the hidden gradient is summed over it.

Counterpart of ``areno/engine/runtime/logprobs.py:23-235`` (which materialises an fp32
probability shard per chunk for backward).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import gemm
from ..ops import logprob as lp_ops
from ..parallel.context import get_context


def _softcap(logits, cap):
    return (torch.tanh(logits.float() / cap) * cap).to(logits.dtype)


class _LMHeadLogprobs(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, chunk, vocab_start, valid_local, tp_group, need_entropy, softcap=0.0):
        rows = hidden.shape[0]
        lp = torch.empty(rows, dtype=torch.float32, device=hidden.device)
        lse = torch.empty_like(lp)
        ex = torch.empty_like(lp)
        # When a backward will follow and the device has room, the bf16 logits of each chunk are kept for it
        # (1.2 GB for 4096 rows of a 152 k vocabulary) instead of being recomputed: one LM-head GEMM less per
        # micro-batch.  Under memory pressure they are dropped and backward recomputes them as before.
        keep = not softcap and _keep_logits(bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1]), hidden, weight, rows)
        kept = [] if keep else None
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            if kept is None:
                # nothing to keep: the GEMM epilogue reduces every tile to the row statistics, no logits tensor exists
                stats = lp_ops.fused_head_stats(hidden[r0:r1], weight, targets[r0:r1], vocab_start, valid_local, softcap)
            else:
                logits = gemm.gemm(hidden[r0:r1], weight)
                stats = lp_ops._stats(logits[:, :valid_local], targets[r0:r1], vocab_start)
                kept.append(logits)
            a, b, c = lp_ops._combine(stats, tp_group)
            lp[r0:r1], lse[r0:r1], ex[r0:r1] = a, b, c
        ctx.kept_logits = kept
        ctx.save_for_backward(hidden, weight, targets, lse, ex)
        ctx.args = (chunk, vocab_start, valid_local, tp_group, need_entropy, float(softcap or 0.0))
        if need_entropy:
            return lp, lse - ex
        return lp

    @staticmethod
    def backward(ctx, dlp, dent=None):
        hidden, weight, targets, lse, ex = ctx.saved_tensors
        chunk, vocab_start, valid_local, tp_group, need_entropy, softcap = ctx.args
        rows = hidden.shape[0]
        dlp = dlp.float().contiguous()
        dent = dent.float().contiguous() if (dent is not None and need_entropy) else None
        dh = torch.empty_like(hidden)
        main_grad = getattr(weight, "main_grad", None)
        dw32 = None
        if main_grad is None:
            dw32 = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        target = main_grad if main_grad is not None else dw32
        kept, ctx.kept_logits = ctx.kept_logits, None     # consumed once: they are overwritten by their gradient
        for ci, r0 in enumerate(range(0, rows, chunk)):
            r1 = min(rows, r0 + chunk)
            h = hidden[r0:r1]
            logits = kept[ci] if kept else gemm.gemm(h, weight)
            if kept:
                kept[ci] = None
            if valid_local < logits.shape[1]:
                logits[:, valid_local:].zero_()
            view = logits[:, :valid_local]
            dcap = None
            if softcap:
                # y = cap tanh(z / cap): the kernel below differentiates with respect to y, then dz = dy (1 - (y / cap)^2)
                y = _softcap(view, softcap)
                dcap = (1.0 - (y.float() / softcap) ** 2).to(view.dtype)
                view.copy_(y)
            lp_ops._lib.call(
                "areno_logprob_bwd", view.data_ptr(), 1, view.stride(0), view.shape[0], valid_local,
                targets[r0:r1].data_ptr(), vocab_start, lse[r0:r1].data_ptr(), ex[r0:r1].data_ptr(),
                dlp[r0:r1].data_ptr(), lp_ops._lib.ptr(dent[r0:r1] if dent is not None else None),
                lp_ops._lib.stream())
            if dcap is not None:
                view.mul_(dcap)
            gemm.gemm(logits, weight, b_mn=True, out=dh[r0:r1])
            gemm.gemm(logits, h, a_mn=True, b_mn=True, out=target, accumulate=True)
        if tp_group is not None and dist.get_world_size(tp_group) > 1:
            dist.all_reduce(dh, group=tp_group)
        dw = None
        if main_grad is not None:
            weight.grad_added_to_main_grad = True
        else:
            dw = dw32.to(weight.dtype)
        return dh, dw, None, None, None, None, None, None, None


def _keep_logits(backward_follows: bool, hidden, weight, rows: int) -> bool:
    """Keep forward logits for backward?  ``ARENO_LOGPROB_KEEP_LOGITS``: ``0`` never, ``1`` always, otherwise when
    they take at most 4 GiB and leave 12 GiB of the device free."""
    if not backward_follows:
        return False
    mode = os.environ.get("ARENO_LOGPROB_KEEP_LOGITS", "auto")
    if mode in ("0", "1"):
        return mode == "1"
    need = rows * weight.shape[0] * 2
    if need > (4 << 30):
        return False
    free, _total = torch.cuda.mem_get_info(hidden.device)
    free += torch.cuda.memory_reserved(hidden.device) - torch.cuda.memory_allocated(hidden.device)
    return free - need > (12 << 30)


def lm_head_logprobs(lm_head, hidden, targets, chunk: int = 4096, need_entropy: bool = False, softcap=None):
    """Log-prob (and entropy) of ``targets`` under ``softmax(lm_head(hidden))``; fp32 ``[rows]``.

    ``lm_head``: a ``VocabParallelLMHead``; ``hidden``: ``[rows, H]``; ``targets``: int64 ``[rows]``.
    """
    ctx = get_context()
    tp_group = ctx.tp_group if ctx.tp_size > 1 else None
    if targets.dtype != torch.int64:
        targets = targets.to(torch.int64)
    if not hidden.is_cuda:
        outs, ents = [], []
        for r0 in range(0, hidden.shape[0], chunk):
            logits = torch.nn.functional.linear(hidden[r0:r0 + chunk], lm_head.weight)[:, : lm_head.valid_local]
            if softcap:
                logits = _softcap(logits, softcap)
            res = _reference_autograd(logits, targets[r0:r0 + chunk], lm_head.vocab_start, tp_group, need_entropy)
            if need_entropy:
                outs.append(res[0])
                ents.append(res[1])
            else:
                outs.append(res)
        if need_entropy:
            return torch.cat(outs), torch.cat(ents)
        return torch.cat(outs)
    hidden = hidden.contiguous()
    return _LMHeadLogprobs.apply(hidden, lm_head.weight, targets.contiguous(), chunk, lm_head.vocab_start,
                                 lm_head.valid_local, tp_group, need_entropy, float(softcap or 0.0))


def _reference_autograd(logits, targets, vocab_start, tp_group, need_entropy):
    """Differentiable fp32 restatement (CPU); single-shard only unless tp_group is given."""
    x = logits.float()
    if tp_group is None:
        logp = torch.log_softmax(x, -1)
        lp = logp.gather(-1, (targets - vocab_start).clamp(0, x.shape[-1] - 1)[:, None]).squeeze(-1)
        if need_entropy:
            return lp, -(logp.exp() * logp).sum(-1)
        return lp
    return _VocabParallelLogprobsCPU.apply(x, targets, vocab_start, tp_group, need_entropy)


class _VocabParallelLogprobsCPU(torch.autograd.Function):
    """Gloo-friendly vocab-parallel selected log-prob with exact backward (for CPU multi-rank tests)."""

    @staticmethod
    def forward(ctx, x, targets, vocab_start, tp_group, need_entropy):
        res = lp_ops.selected_logprobs_reference(x, targets, vocab_start, tp_group, True)
        lp, ent = res
        m = x.max(-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=tp_group)
        s = torch.exp(x - m[:, None]).sum(-1)
        dist.all_reduce(s, group=tp_group)
        lse = m + torch.log(s)
        ctx.save_for_backward(x, targets, lse, lse - ent)
        ctx.vocab_start = vocab_start
        ctx.need_entropy = need_entropy
        return (lp, ent) if need_entropy else lp

    @staticmethod
    def backward(ctx, dlp, dent=None):
        x, targets, lse, ex = ctx.saved_tensors
        p = torch.exp(x - lse[:, None])
        g = -dlp[:, None] * p
        local = targets - ctx.vocab_start
        inside = (local >= 0) & (local < x.shape[-1])
        rows = torch.nonzero(inside).squeeze(-1)
        g[rows, local[rows]] += dlp[rows]
        if dent is not None and ctx.need_entropy:
            g = g - dent[:, None] * p * (x - ex[:, None])
        return g, None, None, None, None
