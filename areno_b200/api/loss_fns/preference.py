"""DPO and SFT objectives (``areno/api/loss_fns/dpo.py:42-74``, ``sft.py:46-57`` in the reference)."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .layout import response_layout, sequence_sum


def dpo_loss_fn(data_pack, logprobs, *, beta: float = 0.1, label_smoothing: float = 0.0):
    """Pairwise logistic loss on summed response log-probs; rows alternate chosen, rejected."""
    beta, label_smoothing = float(beta), float(label_smoothing)
    lay = response_layout(data_pack, logprobs, need_ref_logprobs=True, need_sequences=True)
    n = int(lay.num_sequences) if lay.packed else int(logprobs.shape[0])
    if n % 2 != 0:
        raise ValueError("DPO requires an even number of sequences per microbatch")
    if lay.ref_logprobs is None:
        raise ValueError("DPO requires ref_logprobs in the data pack")
    policy = sequence_sum(logprobs, lay)
    ref = sequence_sum(lay.ref_logprobs.to(logprobs.dtype), lay)
    margin = beta * ((policy[0::2] - policy[1::2]) - (ref[0::2] - ref[1::2]))
    losses = -(1.0 - label_smoothing) * F.logsigmoid(margin) - label_smoothing * F.logsigmoid(-margin)
    loss = losses.mean()
    chosen_r = beta * (policy[0::2] - ref[0::2]).detach()
    rejected_r = beta * (policy[1::2] - ref[1::2]).detach()
    return loss, {
        "dpo_loss": loss.detach(),
        "total_loss": loss.detach(),
        "dpo_accuracy": (margin > 0).float().mean().detach(),
        "dpo_margin": margin.mean().detach(),
        "dpo_reward_margin": (chosen_r - rejected_r).mean(),
        "dpo_chosen_reward": chosen_r.mean(),
        "dpo_rejected_reward": rejected_r.mean(),
        "dpo_response_len": lay.response_len.to(logprobs.dtype).clamp(min=1).mean().detach(),
    }


def sft_loss_fn(data_pack, logprobs):
    """Negative log-likelihood of the non-prompt target tokens.  When the trainer annotates the pack
    with ``_sft_total_target_tokens`` the mean is taken over the whole accumulation group."""
    if "packed_response_mask" in data_pack:
        mask = data_pack["packed_response_mask"].to(device=logprobs.device).to(logprobs.dtype)
    else:
        mask = (~data_pack["prompt_mask"][:, 1:]).to(device=logprobs.device, dtype=logprobs.dtype)
        if "loss_mask" in data_pack:
            mask = mask * data_pack["loss_mask"][:, 1:].to(device=logprobs.device, dtype=logprobs.dtype)
    count = mask.sum().clamp_min(1)
    total_lp = (logprobs * mask).sum()
    group_total = data_pack.get("_sft_total_target_tokens")
    if group_total is None:
        loss = -(total_lp / count)
    else:
        denom = torch.as_tensor(group_total, device=logprobs.device, dtype=logprobs.dtype).clamp_min(1)
        scale = torch.as_tensor(data_pack.get("_sft_grad_scale", 1), device=logprobs.device, dtype=logprobs.dtype)
        loss = -(total_lp / denom) * scale
    return loss, {"sft_loss": loss.detach(), "sft_target_tokens": count.detach(), "sft_logprob_mean": (-loss).detach()}
