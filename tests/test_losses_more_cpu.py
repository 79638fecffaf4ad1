"""More of the loss functions on the CPU: loss masks, padded against packed layouts, the SFT token mean over an
accumulation group, preference pairs with label smoothing, argument errors, gradients that stop at masked tokens, and
GAE corner cases.  Behaviours follow the reference's ``tests/test_more_losses_cpu.py`` and
``tests/test_losses_rewards_cpu.py``."""

from __future__ import annotations

import math

import pytest
import torch

from areno_b200.api import loss_fns
from areno_b200.api.advantages import _compute_gae_python, compute_gae
from areno_b200.api.backend.native import annotate_sft_token_mean_packs, sft_target_token_count
from areno_b200.api.loss_fns.layout import masked_mean, response_layout, sequence_sum
from areno_b200.api.models import TrainSequence
from areno_b200.api.rewards import compute_group_advantages


def _padded():
    """Three rows of width 6: response tokens at columns 2-4, 1-2 and 3; row 0 has one response token masked out."""
    prompt = torch.tensor([[1, 1, 0, 0, 0, 1], [1, 0, 0, 1, 1, 1], [1, 1, 1, 0, 1, 1]], dtype=torch.bool)
    loss_mask = ~prompt
    loss_mask[0, 3] = False
    g = torch.Generator().manual_seed(0)
    return {"prompt_mask": prompt, "loss_mask": loss_mask,
            "logprobs": -torch.rand(3, 6, generator=g), "advantages": torch.randn(3, 6, generator=g),
            "ref_logprobs": -torch.rand(3, 6, generator=g)}


def _as_packed(pack, lp):
    """The same response tokens as flat per-action vectors (what the engine's packed batches look like)."""
    resp = ~pack["prompt_mask"][:, 1:]
    keep = pack["loss_mask"][:, 1:][resp] if "loss_mask" in pack else torch.ones(int(resp.sum()), dtype=torch.bool)
    rows = torch.arange(resp.shape[0])[:, None].expand_as(resp)[resp]
    packed = {"packed_response_mask": keep, "packed_logprobs": pack["logprobs"][:, 1:][resp],
              "packed_advantages": pack["advantages"][:, 1:][resp], "packed_seq_ids": rows,
              "packed_num_sequences": resp.shape[0]}
    if "ref_logprobs" in pack:
        packed["packed_ref_logprobs"] = pack["ref_logprobs"][:, 1:][resp]
    return packed, lp[resp]


def _lp(seed=1):
    return -torch.rand(3, 5, generator=torch.Generator().manual_seed(seed))


# ------------------------------------------------------------------------------------------------------ layout

def test_layout_masks_prompt_padding_and_loss_mask():
    pack = _padded()
    lay = response_layout(pack, _lp(), need_old_logprobs=True, need_advantages=True, need_ref_logprobs=True)
    assert lay.response_mask.tolist() == [[0, 1, 0, 1, 0], [1, 1, 0, 0, 0], [0, 0, 1, 0, 0]]
    assert float(lay.valid_count) == 5 and lay.response_len.tolist() == [2, 2, 1] and not lay.packed
    assert torch.equal(lay.old_logprobs, pack["logprobs"][:, 1:]) and torch.equal(lay.ref_logprobs, pack["ref_logprobs"][:, 1:])
    ones = torch.ones(3, 5)
    assert sequence_sum(ones, lay).tolist() == [2, 2, 1] and float(masked_mean(ones * 3, lay)) == 3.0
    empty = {"prompt_mask": torch.ones(1, 4, dtype=torch.bool)}
    lay0 = response_layout(empty, torch.zeros(1, 3))
    assert float(lay0.valid_count) == 1 and lay0.response_len.tolist() == [1]          # never divide by zero


def test_packed_layout_needs_sequence_ids_for_per_sequence_sums():
    pack = _padded()
    packed, flat = _as_packed(pack, _lp())
    lay = response_layout(packed, flat)
    assert lay.packed and float(lay.valid_count) == 5
    with pytest.raises(ValueError, match="seq_ids"):
        sequence_sum(flat, lay)
    lay = response_layout(packed, flat, need_sequences=True)
    assert lay.response_len.tolist() == [2, 2, 1] and lay.num_sequences == 3


# ------------------------------------------------------------------------------------------------ policy losses

@pytest.mark.parametrize("fn,kw", [
    (loss_fns.grpo_loss_fn, dict(clip_eps=0.2, use_rollout_logprobs=True)),
    (loss_fns.grpo_loss_fn, dict(clip_eps=0.2)),
    (loss_fns.gspo_loss_fn, dict(clip_eps=0.05, use_rollout_logprobs=True)),
    (loss_fns.ppo_loss_fn, dict(clip_eps=0.2, use_kl_loss=True, kl_loss_coef=0.1)),
])
def test_padded_and_packed_batches_give_the_same_loss_and_gradients(fn, kw):
    pack, lp = _padded(), _lp()
    a = lp.clone().requires_grad_(True)
    loss_a, stats_a = fn(pack, a, **kw)
    loss_a.backward()
    packed, flat = _as_packed(pack, lp)
    b = flat.clone().requires_grad_(True)
    loss_b, stats_b = fn(packed, b, **kw)
    loss_b.backward()
    assert math.isclose(float(loss_a.detach()), float(loss_b.detach()), rel_tol=1e-5, abs_tol=1e-7)
    resp = ~pack["prompt_mask"][:, 1:]
    assert torch.allclose(a.grad[resp], b.grad, atol=1e-6)
    assert torch.count_nonzero(a.grad[~resp]) == 0
    assert math.isclose(float(stats_a["advantage_mean"]), float(stats_b["advantage_mean"]), rel_tol=1e-5, abs_tol=1e-7)


def test_masked_response_tokens_get_no_gradient():
    pack, lp = _padded(), _lp()
    for fn in (loss_fns.grpo_loss_fn, loss_fns.gspo_loss_fn, loss_fns.ppo_loss_fn, loss_fns.sft_loss_fn):
        x = lp.clone().requires_grad_(True)
        fn(pack, x)[0].backward()
        assert float(x.grad[0, 2]) == 0.0 and float(x.grad[0, 1]) != 0.0, fn.__name__


def test_policy_statistics_are_detached_scalars():
    pack, lp = _padded(), _lp().requires_grad_(True)
    for fn in (loss_fns.grpo_loss_fn, loss_fns.gspo_loss_fn, loss_fns.ppo_loss_fn):
        loss, stats = fn(pack, lp)
        assert loss.requires_grad and all(not v.requires_grad and v.numel() == 1 for v in stats.values())
        assert math.isclose(float(stats["total_loss"]), float(loss), rel_tol=1e-6)
    _, stats = loss_fns.grpo_loss_fn(pack, lp)
    for key in ("response_len", "rollout_logprobs_mean", "train_logprobs_mean", "logp_diff_mean", "logp_abs_diff_mean"):
        assert key in stats
    assert math.isclose(float(stats["response_len"]), 5 / 3, rel_tol=1e-6)


def test_ppo_reports_clip_fractions_and_refuses_unknown_kl_estimators():
    pack, lp = _padded(), _lp()
    pack["logprobs"] = torch.zeros(3, 6)
    lp = torch.full((3, 5), -1.0)                                   # ratio e^-1 everywhere: below the lower clip
    _, stats = loss_fns.ppo_loss_fn(pack, lp, clip_eps=0.2)
    lay = response_layout(pack, lp, need_advantages=True)
    neg_share = float(masked_mean((lay.advantages < 0).float(), lay))
    assert 0.0 <= float(stats["pg_clipfrac"]) <= 1.0 and float(stats["pg_clipfrac"]) >= neg_share - 1e-6
    assert math.isclose(float(stats["ppo_kl"]), 1.0, rel_tol=1e-6) and float(stats["kl_coef"]) == 0.0
    with pytest.raises(NotImplementedError, match="kl_loss_type"):
        loss_fns.ppo_loss_fn(pack, lp, kl_loss_type="reverse")


def test_ppo_without_reference_logprobs_penalises_against_the_rollout_policy():
    pack, lp = _padded(), _lp()
    del pack["ref_logprobs"]
    total, stats = loss_fns.ppo_loss_fn(pack, lp, use_kl_loss=True, kl_loss_coef=1.0, kl_loss_type="abs")
    lay = response_layout(pack, lp, need_old_logprobs=True)
    assert math.isclose(float(stats["kl_loss"]), float(masked_mean((lp - lay.old_logprobs).abs(), lay)), rel_tol=1e-5)
    assert math.isclose(float(total), float(stats["policy_loss"]) + float(stats["kl_loss"]), rel_tol=1e-5)


# ------------------------------------------------------------------------------------------------ SFT and DPO

def test_sft_counts_only_unmasked_response_tokens():
    pack, lp = _padded(), _lp()
    loss, stats = loss_fns.sft_loss_fn(pack, lp)
    lay = response_layout(pack, lp)
    assert float(stats["sft_target_tokens"]) == 5
    assert math.isclose(float(loss), -float((lp * lay.response_mask).sum()) / 5, rel_tol=1e-6)
    no_mask = {"prompt_mask": pack["prompt_mask"]}
    assert float(loss_fns.sft_loss_fn(no_mask, lp)[1]["sft_target_tokens"]) == 6
    packed, flat = _as_packed(pack, lp)
    assert math.isclose(float(loss_fns.sft_loss_fn(packed, flat)[0]), float(loss), rel_tol=1e-6)


def test_sft_mean_over_an_accumulation_group_weights_tokens_equally():
    """Two micro-batches of 5 and 1 target tokens, accumulated: the optimizer averages the micro-batch losses, so each
    is scaled to make that average the mean over all 6 tokens."""
    lp_a, lp_b = _lp(2), _lp(3)
    a, b = _padded(), {"prompt_mask": torch.tensor([[1, 1, 1, 0, 1, 1]] * 3, dtype=torch.bool)[:1]}
    lp_b = lp_b[:1]
    packs = [a, b]
    annotate_sft_token_mean_packs(packs, [5, 1], gradient_accumulation_steps=None)
    assert a["_sft_total_target_tokens"] == 6 and b["_sft_grad_scale"] == 2
    losses = [loss_fns.sft_loss_fn(p, x)[0] for p, x in zip(packs, (lp_a, lp_b))]
    lay_a = response_layout(a, lp_a)
    want = -(float((lp_a * lay_a.response_mask).sum()) + float(lp_b[0, 2])) / 6
    assert math.isclose(float(sum(losses)) / 2, want, rel_tol=1e-6)
    # groups of two micro-batches each; a short tail group
    packs3 = [{}, {}, {}]
    annotate_sft_token_mean_packs(packs3, [4, 2, 7], gradient_accumulation_steps=2)
    assert [(p["_sft_total_target_tokens"], p["_sft_grad_scale"]) for p in packs3] == [(6, 2), (6, 2), (7, 1)]
    annotate_sft_token_mean_packs([], [], gradient_accumulation_steps=2)


def test_sft_target_count_from_sequences():
    seqs = [TrainSequence(tokens=[1, 2, 3, 4], prompt_mask=[True, True, False, False]),
            TrainSequence(tokens=[1, 2, 3], prompt_mask=[False, False, False], loss_mask=[True, False, True]),
            TrainSequence(tokens=[1], prompt_mask=[False])]
    assert sft_target_token_count(seqs) == 2 + 1 + 0          # position 0 is never a target


def test_dpo_prefers_the_chosen_row_and_label_smoothing_mixes_both_directions():
    prompt = torch.tensor([[1, 0, 0, 1], [1, 0, 0, 0]], dtype=torch.bool)
    pack = {"prompt_mask": prompt, "ref_logprobs": torch.zeros(2, 4)}
    good = torch.tensor([[-0.1, -0.1, -9.0], [-2.0, -2.0, -2.0]], requires_grad=True)
    loss, stats = loss_fns.dpo_loss_fn(pack, good, beta=0.5)
    margin = 0.5 * ((-0.2) - (-6.0))
    assert math.isclose(float(loss), -math.log(1 / (1 + math.exp(-margin))), rel_tol=1e-5)
    assert float(stats["dpo_accuracy"]) == 1.0 and math.isclose(float(stats["dpo_margin"]), margin, rel_tol=1e-6)
    assert math.isclose(float(stats["dpo_chosen_reward"]), -0.1, rel_tol=1e-5)
    assert math.isclose(float(stats["dpo_rejected_reward"]), -3.0, rel_tol=1e-5)
    loss.backward()
    assert float(good.grad[0, 0]) < 0 < float(good.grad[1, 0]) and float(good.grad[0, 2]) == 0.0   # raise chosen, lower rejected
    smooth, _ = loss_fns.dpo_loss_fn(pack, good.detach(), beta=0.5, label_smoothing=0.25)
    want = -0.75 * math.log(1 / (1 + math.exp(-margin))) - 0.25 * math.log(1 / (1 + math.exp(margin)))
    assert math.isclose(float(smooth), want, rel_tol=1e-5)


def test_dpo_argument_errors_and_packed_pairs():
    prompt = torch.tensor([[1, 0, 0]] * 3, dtype=torch.bool)
    with pytest.raises(ValueError, match="even number"):
        loss_fns.dpo_loss_fn({"prompt_mask": prompt, "ref_logprobs": torch.zeros(3, 3)}, torch.zeros(3, 2))
    with pytest.raises(ValueError, match="ref_logprobs"):
        loss_fns.dpo_loss_fn({"prompt_mask": prompt[:2]}, torch.zeros(2, 2))
    packed = {"packed_response_mask": torch.ones(5), "packed_seq_ids": torch.tensor([0, 0, 1, 1, 1]),
              "packed_num_sequences": 2, "packed_ref_logprobs": torch.tensor([-1.0, -1.0, -1.0, -1.0, -1.0])}
    lp = torch.tensor([-0.5, -0.5, -2.0, -2.0, -2.0])
    loss, stats = loss_fns.dpo_loss_fn(packed, lp, beta=1.0)
    margin = (-1.0 - -6.0) - (-2.0 - -3.0)                      # sums per sequence, not means
    assert math.isclose(float(stats["dpo_margin"]), margin, rel_tol=1e-6)
    assert math.isclose(float(stats["dpo_response_len"]), 2.5, rel_tol=1e-6)
    packed["packed_num_sequences"] = 3
    packed["packed_seq_ids"] = torch.tensor([0, 0, 1, 1, 2])
    with pytest.raises(ValueError, match="even number"):
        loss_fns.dpo_loss_fn(packed, lp)


# -------------------------------------------------------------------------------------------------- advantages

def test_group_advantages_are_standardised_and_constant_groups_give_zero():
    adv = compute_group_advantages([2.0, 4.0, 6.0])
    assert math.isclose(sum(adv), 0.0, abs_tol=1e-6) and math.isclose(adv[2], -adv[0], rel_tol=1e-6) and adv[1] == 0.0
    assert compute_group_advantages([3.0]) == [0.0] and compute_group_advantages([]) == []
    assert compute_group_advantages([1.0, 1.0]) == [0.0, 0.0]


def test_gae_terminal_reward_and_length_check():
    adv, ret = _compute_gae_python([0.0, 0.0, 1.0], [0.0, 0.0, 0.0], gamma=1.0, lam=1.0)
    assert adv == [1.0, 1.0, 1.0] and ret == [1.0, 1.0, 1.0]                  # undiscounted: every step sees the reward
    adv, _ = _compute_gae_python([0.0, 1.0], [0.5, 0.5], gamma=0.5, lam=0.0)
    assert adv == [0.0 + 0.5 * 0.5 - 0.5, 1.0 - 0.5]                           # lam 0: one-step TD errors
    assert compute_gae([], [], gamma=0.9, lam=0.9) == ([], [])
    with pytest.raises(ValueError, match="one value per reward"):
        _compute_gae_python([1.0], [0.1, 0.2], gamma=0.9, lam=0.9)


def test_losses_are_importable_from_the_reference_module_paths():
    import importlib

    for name in ("grpo", "gspo", "ppo", "dpo", "sft"):
        mod = importlib.import_module(f"areno_b200.api.loss_fns.{name}")
        assert getattr(mod, f"{name}_loss_fn") is getattr(loss_fns, f"{name}_loss_fn")
