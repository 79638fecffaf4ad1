"""Fused token-level clipped policy loss (PPO dual-clip / GRPO family) with analytic gradient.

Returns per-token loss and KL vectors; masked means stay with the caller so that the same
kernel serves token-mean, sequence-mean and global-token-mean reductions.
Math of ``areno/api/loss_fns/ppo.py:42-99`` and ``grpo.py:25-31`` in the reference.
"""

from __future__ import annotations

import torch

from . import _lib

KL_TYPES = {"kl": 0, "k1": 0, "abs": 1, "mse": 2, "k2": 2, "low_var_kl": 3, "k3": 3}


def kl_penalty_reference(logprob, ref_logprob, kl_type):
    if kl_type in ("kl", "k1"):
        return logprob - ref_logprob
    if kl_type == "abs":
        return (logprob - ref_logprob).abs()
    if kl_type in ("mse", "k2"):
        return 0.5 * (logprob - ref_logprob).square()
    if kl_type in ("low_var_kl", "k3"):
        kl = torch.clamp(ref_logprob - logprob, min=-20.0, max=20.0)
        return torch.clamp(torch.exp(kl) - kl - 1.0, min=-10.0, max=10.0)
    raise NotImplementedError(f"unsupported kl_loss_type: {kl_type}")


def policy_loss_tokens_reference(logprobs, old_logprobs, advantages, ref_logprobs, clip_lo, clip_hi, dual_c, kl_type):
    old = logprobs.detach() if old_logprobs is None else old_logprobs
    d = torch.clamp(logprobs - old, -20.0, 20.0)
    ratio = torch.exp(d)
    clipped = torch.clamp(ratio, 1.0 - clip_lo, 1.0 + clip_hi)
    l1, l2 = -ratio * advantages, -clipped * advantages
    lc = torch.maximum(l1, l2)
    flags = (l2 > l1).int()
    if dual_c and dual_c > 0:
        l3 = -advantages * dual_c
        lower = (advantages < 0) & (lc > l3)
        loss = torch.where(advantages < 0, torch.minimum(l3, lc), lc)
        flags = flags | (lower.int() << 1)
    else:
        loss = lc
    kl = None
    if kl_type is not None and ref_logprobs is not None:
        kl = kl_penalty_reference(logprobs, ref_logprobs, kl_type)
    return loss, kl, flags


class _PolicyLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logprobs, old_logprobs, advantages, ref_logprobs, clip_lo, clip_hi, dual_c, kl_code):
        n = logprobs.numel()
        dev = logprobs.device
        lp = logprobs.detach().float().contiguous()
        buf = torch.empty((4, n), dtype=torch.float32, device=dev)
        flags = torch.empty(n, dtype=torch.int32, device=dev)
        old = old_logprobs.float().contiguous() if old_logprobs is not None else None
        ref = ref_logprobs.float().contiguous() if ref_logprobs is not None else None
        adv = advantages.float().contiguous()
        _lib.call("areno_policy_loss", lp.data_ptr(), _lib.ptr(old), adv.data_ptr(), _lib.ptr(ref),
                  buf[0].data_ptr(), buf[1].data_ptr(), buf[2].data_ptr(), buf[3].data_ptr(), flags.data_ptr(), n,
                  float(clip_lo), float(clip_hi), float(dual_c or 0.0), int(kl_code), _lib.stream())
        ctx.save_for_backward(buf)
        ctx.shape = logprobs.shape
        ctx.mark_non_differentiable(flags)
        return buf[0].view(logprobs.shape), buf[1].view(logprobs.shape), flags.view(logprobs.shape)

    @staticmethod
    def backward(ctx, dloss, dkl, _dflags):
        (buf,) = ctx.saved_tensors
        g = dloss.reshape(-1) * buf[2]
        if dkl is not None:
            g = g + dkl.reshape(-1) * buf[3]
        return g.view(ctx.shape), None, None, None, None, None, None, None


def policy_loss_tokens(logprobs, old_logprobs, advantages, ref_logprobs=None, clip_lo=0.2, clip_hi=0.2,
                       dual_c: float = 0.0, kl_type: str | None = None):
    """Per-token (loss, kl, flags).  ``old_logprobs=None`` selects the on-policy surrogate
    (ratio identically 1 in value, gradient ``-A``)."""
    if not logprobs.is_cuda:
        return policy_loss_tokens_reference(logprobs, old_logprobs, advantages, ref_logprobs, clip_lo, clip_hi,
                                            dual_c, kl_type)
    code = KL_TYPES[kl_type] if (kl_type is not None and ref_logprobs is not None) else -1
    loss, kl, flags = _PolicyLoss.apply(logprobs, old_logprobs, advantages, ref_logprobs, clip_lo, clip_hi, dual_c,
                                        code)
    return loss, (kl if code >= 0 else None), flags
