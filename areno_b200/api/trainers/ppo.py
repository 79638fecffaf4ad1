"""PPO with actor / reference / critic (/ reward-model) roles.

Per step (``areno/api/trainers/ppo.py:84-377`` in the reference): score rewards (Python function or
reward role), reference log-probs, actor old log-probs (re-scored with the training kernels, not
taken from rollout), critic values; per-response GAE with the reward on the last response token;
critic update; batch-wide advantage standardisation over loss tokens; actor update (skipped for
the first ``critic_warmup_steps`` steps).  Prompt and agentic rollouts go through one code path:
both are reduced to token rows with response / loss masks.
"""

from __future__ import annotations

import time
from functools import partial

import numpy as np

from ..advantages import compute_gae
from ..models import TrainSequence
from ..rewards import make_reward_record
from ..roles import MissingRoleCapability, ModelRole
from .policy_only import PolicyOnlyTrainer


def summary_stats(name: str, values: list[float]) -> dict[str, float]:
    if not values:
        return {}
    a = np.asarray(values, dtype=np.float64)
    return {f"{name}_mean": float(a.mean()), f"{name}_std": float(a.std()), f"{name}_min": float(a.min()),
            f"{name}_max": float(a.max())}


def normalize_response_advantages(train_batch: list[TrainSequence]) -> None:
    """In place: standardise advantages over all loss tokens of the batch (std floor 1e-6)."""
    def mask_of(seq):
        return seq.loss_mask if seq.loss_mask else [not p for p in seq.prompt_mask]

    vals = [a for seq in train_batch for a, on in zip(seq.advantages, mask_of(seq)) if on]
    if not vals:
        return
    mean, std = float(np.mean(vals)), float(np.std(vals))
    scale = std if std > 1e-6 else 1.0
    for seq in train_batch:
        seq.advantages = [(a - mean) / scale if on else 0.0 for a, on in zip(seq.advantages, mask_of(seq))]


def _floats(values) -> list[float]:
    if hasattr(values, "detach"):
        values = values.detach().float().cpu().tolist()
    return [float(v) for v in values]


class PPOTrainer(PolicyOnlyTrainer):
    def __init__(self, config, *, instance, dataset, reward_fn, loss_fn):
        super().__init__(config, instance=instance, dataset=dataset, reward_fn=reward_fn, loss_fn=loss_fn)
        self.loss_fn = partial(loss_fn, clip_eps=config.clip_eps, clip_ratio_c=config.clip_ratio_c,
                               use_kl_loss=config.use_kl_loss, kl_loss_coef=config.kl_loss_coef,
                               kl_loss_type=config.kl_loss_type)
        self._last_ppo_stats: dict[str, float] = {}
        self.roles = {
            "actor": ModelRole("actor", config.ckpt, trainable=True),
            "ref": ModelRole("ref", config.ref_ckpt or config.ckpt, trainable=False),
            "critic": ModelRole("critic", config.critic_ckpt or config.ckpt, trainable=True,
                                optimizer_lr=float(config.critic_lr)),
        }
        if config.reward_ckpt:
            self.roles["reward"] = ModelRole("reward", config.reward_ckpt, trainable=False)

    def _policy_role_name(self) -> str:
        return "actor"

    def _should_train_policy(self, step: int) -> bool:
        return step >= int(self.config.critic_warmup_steps)

    def _augment_train_stats(self, result):
        if isinstance(result, dict):
            result.update(self._last_ppo_stats)
        return result

    def _prepare(self) -> None:
        for role in self.roles.values():
            self.logger.info("role=%s stage=init_start trainable=%s path=%s", role.name, role.trainable, role.path)
        self.areno.ensure_roles(self.roles)
        for role in self.roles.values():
            self.logger.info("role=%s stage=init_end trainable=%s", role.name, role.trainable)

    # ------------------------------------------------------------ materialise
    def _materialize_train_batch(self, tokenizer, prompt_batch, rollout_results):
        rows, rmasks, lmasks, rollout_rows, records = [], [], [], [], []
        for pi, (item, result) in enumerate(zip(prompt_batch.items, rollout_results)):
            n_p = len(item.input_tokens)
            for si, seq in enumerate(result.sequences):
                n_r = len(seq.resp_tokens)
                tokens = item.input_tokens + seq.resp_tokens
                rows.append(tokens)
                rmasks.append([False] * n_p + [True] * n_r)
                lmasks.append([False] * n_p + [True] * n_r)
                rollout_rows.append([0.0] * n_p + list(seq.resp_logprobs))
                records.append(make_reward_record(
                    prompt=item.prompt, completion=tokenizer.decode(seq.resp_tokens), source_record=item.record,
                    answer=item.solutions, tokens=tokens, logprobs=rollout_rows[-1], loss_mask=lmasks[-1],
                    metadata={"prompt_index": pi, "sample_index": si}))
        rewards = None
        if self.reward_fn is not None:
            t0 = time.perf_counter()
            rewards = [float(self.reward_fn(r)) for r in records]
            self._last_ppo_stats = {"reward_score_time_s": time.perf_counter() - t0}
        else:
            self._last_ppo_stats = {}
        return self._build_ppo_batch(tokenizer, rows, rmasks, lmasks, rollout_rows, rewards, explicit_loss_mask=False)

    def _materialize_agentic_train_batch(self, tokenizer, prompt_batch, agent_batch):
        self._last_ppo_stats = {}
        rewards = [float(r) for r in agent_batch.rewards] if agent_batch.rewards is not None else None
        return self._build_ppo_batch(tokenizer, agent_batch.token_rows, agent_batch.response_masks,
                                     agent_batch.loss_masks, agent_batch.rollout_logprobs, rewards,
                                     explicit_loss_mask=True)

    def _timed(self, key: str, role: str, stage: str, rows: int, fn):
        self.logger.info("role=%s stage=%s_start rows=%d", role, stage, rows)
        t0 = time.perf_counter()
        out = fn()
        self._last_ppo_stats[key] = time.perf_counter() - t0
        self.logger.info("role=%s stage=%s_end rows=%d", role, stage, rows)
        return out

    def _build_ppo_batch(self, tokenizer, rows, rmasks, lmasks, rollout_rows, rewards, *, explicit_loss_mask: bool):
        n = len(rows)
        if rewards is None:
            if "reward" not in self.roles:
                raise MissingRoleCapability("PPO needs a reward function or a --reward-ckpt reward model")
            rewards = _floats(self._timed("reward_score_time_s", "reward", "score", n,
                                          lambda: self.areno.score_rewards("reward", rows)))
            self._last_ppo_stats.update(summary_stats("reward_model_raw_reward", rewards))
        ref_rows = self._timed("ref_logprob_forward_time_s", "ref", "logprob_score", n,
                               lambda: self.areno.score_logprobs("ref", rows))
        old_rows = self._timed("actor_old_logprob_forward_time_s", "actor", "old_logprob_score", n,
                               lambda: self.areno.score_logprobs("actor", rows))
        value_rows = self._timed("critic_value_forward_time_s", "critic", "value_score", n,
                                 lambda: self.areno.score_values("critic", rows))
        eos = getattr(tokenizer, "eos_token_id", None) or 0
        batch: list[TrainSequence] = []
        rollout_lp, ref_all, old_all, diff_all, val_all, ret_all, adv_all = [], [], [], [], [], [], []
        for tokens, rmask, lmask, roll, reward, ref_lp, old_lp, values in zip(rows, rmasks, lmasks, rollout_rows, rewards,
                                                                              ref_rows, old_rows, value_rows):
            if not (len(tokens) == len(rmask) == len(lmask) == len(roll)):
                raise ValueError("PPO batch has misaligned token/mask/logprob rows")
            resp_idx = [i for i, r in enumerate(rmask) if r]
            if not resp_idx or not any(lmask[i] for i in resp_idx):
                continue
            # A multi-turn agentic row has several assistant spans with tool results between them, so the response
            # positions need not be contiguous: every per-action signal is gathered by position (the reference
            # slices ``[first, first + count)``, which is the same thing only for a single span).
            n_r = len(resp_idx)
            if len(old_lp) < len(tokens) or len(ref_lp) < len(tokens):
                raise ValueError("actor returned misaligned old logprobs")
            if len(values) < len(tokens) or resp_idx[0] < 1:
                raise ValueError("critic returned misaligned token values")
            old_lp, ref_lp, values = _floats(old_lp), _floats(ref_lp), _floats(values)
            act_old = [old_lp[i] for i in resp_idx]
            act_values = [values[i - 1] for i in resp_idx]          # the value before token i is generated
            token_rewards = [0.0] * n_r
            token_rewards[-1] = float(reward)
            adv, ret = compute_gae(token_rewards, act_values, gamma=self.config.gamma, lam=self.config.lam)
            adv, ret = _floats(adv), _floats(ret)
            full_adv, full_ret, full_val = [0.0] * len(tokens), [0.0] * len(tokens), [0.0] * len(tokens)
            full_old = [0.0] * len(tokens)
            for rel, ti in enumerate(resp_idx):
                if lmask[ti]:
                    full_adv[ti] = adv[rel]
                full_ret[ti] = ret[rel]
                full_val[ti] = act_values[rel]
                full_old[ti] = act_old[rel]
            roll_resp = [float(roll[i]) for i in resp_idx]
            rollout_lp.extend(lp for lp, i in zip(roll_resp, resp_idx) if lmask[i])
            old_all.extend(act_old)
            diff_all.extend(o - r for o, r in zip(act_old, roll_resp))
            ref_all.extend(ref_lp[i] for i in resp_idx)
            val_all.extend(act_values)
            ret_all.extend(ret)
            adv_all.extend(adv)
            batch.append(TrainSequence(
                prompt_mask=[not r for r in rmask], loss_mask=list(lmask) if explicit_loss_mask else [],
                tokens=list(tokens), logprobs=full_old,
                advantages=full_adv, returns=full_ret, values=full_val, ref_logprobs=ref_lp[:len(tokens)],
                reward=float(reward), eos_token_id=eos))
        if batch:
            stats = self._timed("critic_train_time_s", "critic", "train", len(batch), lambda: self.areno.train_values(
                "critic", batch, self.config.mini_bs, self.config.gradient_accumulation_steps,
                cliprange_value=self.config.value_clip_eps, value_loss_coef=self.config.value_loss_coef))
            if stats:
                self._last_ppo_stats.update({k: float(v) for k, v in stats.items() if isinstance(v, (int, float))})
                if "critic_value_loss" in stats:
                    self.logger.info("role=critic metric=value_loss value=%.6f", float(stats["critic_value_loss"]))
            for name, vals in (("ref_logprob", ref_all), ("old_logprob", old_all),
                               ("old_rollout_logprob_diff", diff_all), ("critic_value", val_all), ("return", ret_all),
                               ("gae_advantage", adv_all)):
                self._last_ppo_stats.update(summary_stats(name, vals))
            normalize_response_advantages(batch)
            norm = [a for s in batch for a, on in zip(s.advantages, s.loss_mask or [not p for p in s.prompt_mask]) if on]
            self._last_ppo_stats.update(summary_stats("normalized_advantage", norm))
        return batch, list(rewards), rollout_lp


__all__ = ["PPOTrainer", "MissingRoleCapability"]
