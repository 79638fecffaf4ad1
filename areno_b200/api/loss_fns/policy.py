"""Policy-gradient losses: GSPO (sequence ratio), GRPO (token ratio), PPO (dual clip + KL).

GSPO and GRPO keep the reference default of the on-policy surrogate
``log r = logp - logp.detach()`` - the ratio is 1 in value, the clip never binds on the single
update per batch, and rollout log-probs only feed diagnostics
(``areno/api/loss_fns/gspo.py:28-44``, ``grpo.py:25-31``).  Pass ``use_rollout_logprobs=True`` for
the true importance ratio against the rollout policy.  The token-level losses run the fused
``policy_loss`` kernel on CUDA.
"""

from __future__ import annotations

import torch

from ...ops.policy_loss import kl_penalty_reference, policy_loss_tokens
from .layout import masked_mean, response_layout, sequence_sum


def _ratio_stats(ratio, layout, dev):
    valid = ratio[layout.response_mask.bool()]
    mean = valid.mean().detach() if valid.numel() else ratio.mean().detach()
    std = valid.std().detach() if valid.numel() > 1 else torch.zeros((), device=dev)
    return mean, std


def _rollout_diagnostics(logprobs, layout):
    train = logprobs.detach()
    diff = layout.old_logprobs - train
    return {
        "response_len": layout.response_len.mean().detach(),
        "rollout_logprobs_mean": masked_mean(layout.old_logprobs, layout).detach(),
        "train_logprobs_mean": masked_mean(train, layout).detach(),
        "logp_diff_mean": masked_mean(diff, layout).detach(),
        "logp_abs_diff_mean": masked_mean(diff.abs(), layout).detach(),
    }


def gspo_loss_fn(data_pack, logprobs, *, clip_eps: float = 3e-4, use_rollout_logprobs: bool = False):
    """Sequence-level clipped objective: one ratio per response (mean token log-ratio)."""
    clip_eps = float(clip_eps)
    lay = response_layout(data_pack, logprobs, need_old_logprobs=True, need_advantages=True, need_sequences=True)
    anchor = lay.old_logprobs if use_rollout_logprobs else logprobs.detach()
    seq_log_ratio = sequence_sum(logprobs - anchor, lay) / lay.response_len
    seq_ratio = torch.exp(seq_log_ratio)
    clipped = torch.clamp(seq_ratio, 1.0 - clip_eps, 1.0 + clip_eps)
    seq_adv = sequence_sum(lay.advantages, lay) / lay.response_len
    loss = (-torch.min(seq_ratio * seq_adv, clipped * seq_adv)).mean()
    stats = {
        "policy_loss": loss.detach(),
        "total_loss": loss.detach(),
        "ratio_mean": seq_ratio.mean().detach(),
        "ratio_std": seq_ratio.std(unbiased=False).detach(),
        "advantage_mean": seq_adv.mean().detach(),
    }
    stats.update(_rollout_diagnostics(logprobs, lay))
    return loss, stats


def grpo_loss_fn(data_pack, logprobs, *, clip_eps: float = 0.2, use_rollout_logprobs: bool = False):
    """Token-level clipped objective averaged over all response tokens of the micro-batch."""
    clip_eps = float(clip_eps)
    lay = response_layout(data_pack, logprobs, need_old_logprobs=True, need_advantages=True, need_sequences=True)
    old = lay.old_logprobs if use_rollout_logprobs else None
    per_token, _, _ = policy_loss_tokens(logprobs, old, lay.advantages, None, clip_eps, clip_eps, 0.0, None)
    loss = (per_token * lay.response_mask).sum() / lay.valid_count
    with torch.no_grad():
        ratio = torch.exp(logprobs.detach() - (old if old is not None else logprobs.detach()))
        r_mean, r_std = _ratio_stats(ratio, lay, logprobs.device)
    stats = {
        "policy_loss": loss.detach(),
        "total_loss": loss.detach(),
        "ratio_mean": r_mean,
        "ratio_std": r_std,
        "advantage_mean": masked_mean(lay.advantages, lay).detach(),
    }
    stats.update(_rollout_diagnostics(logprobs, lay))
    return loss, stats


def ppo_loss_fn(data_pack, logprobs, *, clip_eps: float = 0.2, clip_ratio_c: float = 3.0, use_kl_loss: bool = False,
                kl_loss_coef: float = 0.001, kl_loss_type: str = "low_var_kl"):
    """PPO actor loss with real old log-probs, dual clip for negative advantages and an optional
    KL-to-reference penalty (estimators kl / abs / mse / low_var_kl)."""
    clip_eps, clip_ratio_c, kl_loss_coef = float(clip_eps), float(clip_ratio_c), float(kl_loss_coef)
    if kl_loss_type not in ("kl", "k1", "abs", "mse", "k2", "low_var_kl", "k3"):
        raise NotImplementedError(f"unsupported PPO kl_loss_type: {kl_loss_type}")
    lay = response_layout(data_pack, logprobs, need_old_logprobs=True, need_advantages=True, need_ref_logprobs=True)
    ref = lay.old_logprobs if lay.ref_logprobs is None else lay.ref_logprobs
    per_token, kl_tok, flags = policy_loss_tokens(logprobs, lay.old_logprobs, lay.advantages, ref, clip_eps, clip_eps,
                                                  clip_ratio_c, kl_loss_type)
    if kl_tok is None:
        kl_tok = kl_penalty_reference(logprobs, ref, kl_loss_type)
    policy_loss = masked_mean(per_token, lay)
    kl = masked_mean(kl_tok, lay)
    total = policy_loss + (kl_loss_coef * kl if use_kl_loss else 0.0)
    with torch.no_grad():
        neg_kl = torch.clamp(logprobs.detach() - lay.old_logprobs, -20.0, 20.0)
        ratio = torch.exp(neg_kl)
        r_mean, r_std = _ratio_stats(ratio, lay, logprobs.device)
        upper = (flags & 1).float()
        lower = ((flags >> 1) & 1).float()
    return total, {
        "policy_loss": policy_loss.detach(),
        "kl_loss": kl.detach(),
        "kl_coef": torch.tensor(kl_loss_coef if use_kl_loss else 0.0, device=logprobs.device),
        "pg_clipfrac": masked_mean(upper, lay).detach(),
        "pg_clipfrac_lower": masked_mean(lower, lay).detach(),
        "ppo_kl": masked_mean(-neg_kl, lay).detach(),
        "total_loss": total.detach(),
        "ratio_mean": r_mean,
        "ratio_std": r_std,
        "advantage_mean": masked_mean(lay.advantages, lay).detach(),
    }
