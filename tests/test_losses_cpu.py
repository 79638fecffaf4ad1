"""Loss functions, advantages and rewards against hand-written formulas (padded and packed layouts)."""

from __future__ import annotations

import math

import torch

from areno_b200.api import loss_fns
from areno_b200.api.advantages import compute_gae
from areno_b200.api.rewards import compute_group_advantages


def _padded_pack():
    prompt_mask = torch.tensor([[1, 1, 0, 0, 0, 1], [1, 0, 0, 1, 1, 1]], dtype=torch.bool)
    prompt_mask[0, 5] = True      # padding counts as prompt
    pack = {"prompt_mask": prompt_mask, "logprobs": torch.tensor([[0, 0, -1.0, -2.0, -0.5, 0], [0, -1.5, -0.3, 0, 0, 0]]),
            "advantages": torch.tensor([[0, 0, 1.0, 1.0, 1.0, 0], [0, -2.0, -2.0, 0, 0, 0]])}
    return pack


def test_grpo_is_on_policy_surrogate_with_unit_ratio():
    pack = _padded_pack()
    lp = torch.tensor([[-9, -1.1, -2.2, -0.4, -9], [-1.4, -0.2, -9, -9, -9]], requires_grad=True)   # per action: [B, T-1]
    loss, stats = loss_fns.grpo_loss_fn(pack, lp, clip_eps=0.2)
    mask = (~pack["prompt_mask"][:, 1:]).float()
    adv = pack["advantages"][:, 1:]
    assert math.isclose(float(loss), float(-(adv * mask).sum() / mask.sum()), rel_tol=1e-6)   # ratio == 1
    loss.backward()
    # d/dlogp of -(ratio * A) at ratio 1 is -A / count on response positions, zero elsewhere
    assert torch.allclose(lp.grad, -(adv * mask) / mask.sum(), atol=1e-7)
    assert float(stats["ratio_mean"]) == 1.0
    # against the rollout log-probs the ratio is exp(new - old) and clipping applies
    lp2 = lp.detach().clone().requires_grad_()
    loss2, _ = loss_fns.grpo_loss_fn(pack, lp2, clip_eps=0.2, use_rollout_logprobs=True)
    ratio = torch.exp(lp2.detach() - pack["logprobs"][:, 1:])
    per = -torch.min(ratio * adv, ratio.clamp(0.8, 1.2) * adv)
    assert math.isclose(float(loss2), float((per * mask).sum() / mask.sum()), rel_tol=1e-5)


def test_gspo_sequence_ratio_and_packed_layout_agree():
    pack = _padded_pack()
    lp = torch.tensor([[-9, -1.1, -2.2, -0.4, -9], [-1.4, -0.2, -9, -9, -9]])
    loss, _ = loss_fns.gspo_loss_fn(pack, lp, clip_eps=0.1, use_rollout_logprobs=True)
    mask = (~pack["prompt_mask"][:, 1:]).float()
    old, adv = pack["logprobs"][:, 1:], pack["advantages"][:, 1:]
    n = mask.sum(-1)
    seq_ratio = torch.exp(((lp - old) * mask).sum(-1) / n)
    seq_adv = (adv * mask).sum(-1) / n
    ref = (-torch.min(seq_ratio * seq_adv, seq_ratio.clamp(0.9, 1.1) * seq_adv)).mean()
    assert math.isclose(float(loss), float(ref), rel_tol=1e-6)
    # the packed (varlen) description of the same two responses gives the same loss
    idx = mask.bool()
    packed = {"packed_response_mask": torch.ones(int(mask.sum())), "packed_logprobs": old[idx],
              "packed_advantages": adv[idx], "packed_seq_ids": torch.tensor([0, 0, 0, 1, 1]), "packed_num_sequences": 2}
    loss_p, _ = loss_fns.gspo_loss_fn(packed, lp[idx], clip_eps=0.1, use_rollout_logprobs=True)
    assert math.isclose(float(loss_p), float(ref), rel_tol=1e-6)


def test_ppo_dual_clip_and_kl_estimators():
    pack = _padded_pack()
    pack["ref_logprobs"] = pack["logprobs"] - 0.1
    lp = torch.tensor([[-9, -0.2, -2.6, -0.4, -9], [-3.0, -0.2, -9, -9, -9]])
    mask = (~pack["prompt_mask"][:, 1:]).float()
    old, adv, ref = pack["logprobs"][:, 1:], pack["advantages"][:, 1:], pack["ref_logprobs"][:, 1:]
    cur = lp
    ratio = torch.exp((cur - old).clamp(-20, 20))
    pg = torch.max(-adv * ratio, -adv * ratio.clamp(0.8, 1.2))
    pg = torch.where(adv < 0, torch.min(pg, -adv * 3.0), pg)
    for kind, fn in (("kl", lambda d: d), ("abs", lambda d: d.abs()), ("mse", lambda d: 0.5 * d * d),
                     ("low_var_kl", lambda d: (torch.exp(-d) + d - 1).clamp(-10, 10))):
        total, stats = loss_fns.ppo_loss_fn(pack, lp, clip_eps=0.2, clip_ratio_c=3.0, use_kl_loss=True, kl_loss_coef=0.5,
                                            kl_loss_type=kind)
        kl = fn(cur - ref)
        want = (pg * mask).sum() / mask.sum() + 0.5 * (kl * mask).sum() / mask.sum()
        assert math.isclose(float(total), float(want), rel_tol=1e-5, abs_tol=1e-6), kind
    assert 0.0 < float(stats["pg_clipfrac"]) <= 1.0


def test_dpo_and_sft():
    # two pairs, interleaved chosen / rejected rows
    prompt_mask = torch.tensor([[1, 0, 0], [1, 0, 0], [1, 0, 1], [1, 0, 0]], dtype=torch.bool)
    pack = {"prompt_mask": prompt_mask, "ref_logprobs": torch.tensor([[0, -1.0, -1.0], [0, -1.0, -1.0], [0, -2.0, 0], [0, -1.0, -3.0]])}
    lp = torch.tensor([[-0.5, -0.5], [-1.5, -1.5], [-1.0, 0], [-2.0, -2.0]])
    loss, stats = loss_fns.dpo_loss_fn(pack, lp, beta=0.2)
    mask = (~prompt_mask[:, 1:]).float()
    pol = (lp * mask).sum(-1)
    refs = (pack["ref_logprobs"][:, 1:] * mask).sum(-1)
    margins = 0.2 * ((pol[0::2] - pol[1::2]) - (refs[0::2] - refs[1::2]))
    assert math.isclose(float(loss), float(-torch.nn.functional.logsigmoid(margins).mean()), rel_tol=1e-6)
    assert float(stats["dpo_accuracy"]) == float((margins > 0).float().mean())
    sft, _ = loss_fns.sft_loss_fn({"prompt_mask": prompt_mask[:2]}, lp[:2])
    assert math.isclose(float(sft), float(-(lp[:2]).mean()), rel_tol=1e-6)


def test_advantages():
    adv = compute_group_advantages([1.0, 0.0, 0.0, 1.0])
    assert math.isclose(sum(adv), 0.0, abs_tol=1e-6) and adv[0] > 0 > adv[1]
    assert compute_group_advantages([0.5, 0.5, 0.5]) == [0.0, 0.0, 0.0]
    rewards, values = [0.0, 0.0, 1.0], [0.2, 0.4, 0.6]
    a, r = compute_gae(rewards, values, gamma=0.9, lam=0.8)
    # backward recursion by hand
    d2 = 1.0 - 0.6
    d1 = 0.9 * 0.6 - 0.4
    d0 = 0.9 * 0.4 - 0.2
    a2, a1 = d2, d1 + 0.72 * d2
    a0 = d0 + 0.72 * a1
    assert all(math.isclose(x, y, rel_tol=1e-6) for x, y in zip(a, [a0, a1, a2]))
    assert all(math.isclose(x, y + v, rel_tol=1e-6) for x, y, v in zip(r, [a0, a1, a2], values))
