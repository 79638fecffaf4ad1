"""Rollout -> reward -> train loop for policy-only RL (GSPO / GRPO), prompt-based or agentic.

Semantics of ``areno/api/trainers/policy_only.py:27-557`` in the reference: rollouts run inside a
rollout session; each completion is scored by ``reward_fn(RewardRecord)``; advantages are rewards
normalised within the prompt's sample group and broadcast to the response tokens (prompt positions
carry zero advantage and zero log-prob); agentic trajectories longer than the context limit are
dropped with diagnostics; ``ARENO_LOG_COMPLETIONS=N`` logs the first N completions of a step.
"""

from __future__ import annotations

import asyncio
import os
import time

import numpy as np

from ..models import SamplingParams, TrainSequence
from ..rewards import compute_group_advantages, make_reward_record
from ..tokenizer import configure_chat_template_enable_thinking
from .base import BaseTrainer


class PolicyOnlyTrainer(BaseTrainer):
    def __init__(self, config, *, instance, dataset, reward_fn, loss_fn):
        super().__init__(config, instance=instance, dataset=dataset, reward_fn=reward_fn, loss_fn=loss_fn)
        self._agent_run_fn = None

    # ----------------------------------------------------------------- hooks
    def _policy_role_name(self) -> str:
        return "policy"

    def _should_train_policy(self, step: int) -> bool:
        return True

    def _augment_train_stats(self, result):
        return result

    def _prepare(self) -> None:
        """Called once after ``init`` (PPO loads its roles here)."""

    def _after_rollout(self, train_batch: list[TrainSequence], epoch: int, step: int) -> list[TrainSequence]:
        """Called with the materialised batch before the policy update (PPO scores / trains roles here)."""
        return train_batch

    # ------------------------------------------------------------------ loop
    def _sampling_params(self) -> SamplingParams:
        c = self.config
        return SamplingParams(greedy=c.greedy, temperature=c.temperature, max_new_tokens=c.max_new_tokens,
                              max_context_len=getattr(c, "max_context_len", None), max_prompt_len=c.max_prompt_tokens,
                              top_k=c.top_k, top_p=c.top_p)

    def _fit_initialized(self) -> None:
        tokenizer = self.areno.get_tokenizer()
        configure_chat_template_enable_thinking(tokenizer, getattr(self.config, "chat_template_enable_thinking", None))
        params = self._sampling_params()
        self._prepare()
        step = 0
        for epoch in range(self.config.epochs):
            self.logger.info("epoch=%d stage=epoch_start", epoch)
            for prompt_batch in self.areno.load_prompt_batches(self.dataset, batch_size=self.config.batch_size,
                                                               max_prompt_tokens=self.config.max_prompt_tokens):
                role = self._policy_role_name()
                self.logger.info("epoch=%d step=%d role=%s stage=rollout_start", epoch, step, role)
                if self._agentic_enabled():
                    agent_batch = asyncio.run(self._run_agentic_rollout(params, prompt_batch))
                    self.logger.info("epoch=%d step=%d role=%s stage=rollout_end", epoch, step, role)
                    self._log_agentic_completions(epoch, step, agent_batch)
                    batch, rewards, rollout_lp = self._materialize_agentic_train_batch(tokenizer, prompt_batch, agent_batch)
                else:
                    results = asyncio.run(self._run_prompt_rollout(params, prompt_batch))
                    self.logger.info("epoch=%d step=%d role=%s stage=rollout_end", epoch, step, role)
                    self._log_completions(tokenizer, epoch, step, prompt_batch, results)
                    batch, rewards, rollout_lp = self._materialize_train_batch(tokenizer, prompt_batch, results)
                if rewards:
                    self.logger.info("epoch=%d step=%d metric=reward_mean value=%.6f", epoch, step, float(np.mean(rewards)))
                if rollout_lp:
                    self.logger.info("epoch=%d step=%d metric=rollout_logprob_mean value=%.6f", epoch, step,
                                     float(np.mean(rollout_lp)))
                if batch:
                    batch = self._after_rollout(batch, epoch, step)
                    if not self._should_train_policy(step):
                        result = self._augment_train_stats({"actor_train_skipped": 1.0})
                        self.logger.info("epoch=%d step=%d role=%s stage=train_skip", epoch, step, role)
                        self.logger.info("epoch=%d step=%d train_stats=%s", epoch, step, result)
                        self.areno.finish_step()
                    else:
                        self.logger.info("epoch=%d step=%d role=%s stage=train_start", epoch, step, role)
                        t0 = time.perf_counter()
                        result = self.areno.train(batch, self.loss_fn, mini_bs=self.config.mini_bs,
                                                  gradient_accumulation_steps=self.config.gradient_accumulation_steps)
                        if isinstance(result, dict):
                            result[f"{role}_train_wall_time_s"] = time.perf_counter() - t0
                        result = self._augment_train_stats(result)
                        self.logger.info("epoch=%d step=%d role=%s stage=train_end", epoch, step, role)
                        self.logger.info("epoch=%d step=%d train_stats=%s", epoch, step, result)
                        self._maybe_save(epoch, step)
                step += 1
                if self._reached_max_steps(epoch, step):
                    return
            self.logger.info("epoch=%d stage=epoch_end", epoch)

    # -------------------------------------------------------------- rollouts
    async def _run_prompt_rollout(self, params, prompt_batch):
        async with self.areno.rollout_session(sampling_params=params, proxy=False,
                                              max_running_prompts=self.config.resolved_max_running_prompts()):
            tokens = [item.input_tokens for item in prompt_batch.items]
            return await self.areno.rollout_token_batch_async(tokens, self.config.n_samples, params)

    def _agentic_enabled(self) -> bool:
        return bool(getattr(self.config, "agent_fn", None))

    def _loss_mask_policy(self):
        from ..agentic import LossMaskPolicy

        return LossMaskPolicy(tool_results=bool(getattr(self.config, "train_tool_results", False)))

    def _get_agent_run_fn(self):
        from ..agentic import load_agent_run_fn

        if self._agent_run_fn is None:
            self._agent_run_fn = load_agent_run_fn(self.config.agent_fn)
        return self._agent_run_fn

    async def _run_agentic_rollout(self, params, prompt_batch):
        from ..agentic import AgentBatch, maybe_await

        agent_batch = AgentBatch.from_prompt_batch(prompt_batch, n_samples=self.config.n_samples)
        self.logger.info("agentic rollout batch prompts=%d n_samples=%d expected_requests=%d max_running_prompts=%d",
                         len(agent_batch.records), agent_batch.n_samples, len(agent_batch),
                         self.config.resolved_max_running_prompts())
        async with self.areno.rollout_session(sampling_params=params, loss_mask_policy=self._loss_mask_policy(),
                                              max_running_prompts=self.config.resolved_max_running_prompts(),
                                              timeout_s=self.config.agent_timeout_s) as session:
            await session.sync_rollout_session_async()
            trajectories = await maybe_await(self._get_agent_run_fn()(session, agent_batch))
            if trajectories is None:
                raise RuntimeError("agent run function must return explicit trajectories")
            samples = session.accumulate(self._normalize_trajectories(trajectories))
            samples, dropped, diag = self._filter_overlong(samples, params)
            if len(samples) + dropped != len(agent_batch):
                raise RuntimeError(f"agent rollout produced {len(samples)} trajectories and filtered {dropped}, "
                                   f"expected {len(agent_batch)}")
            if not samples:
                raise RuntimeError(f"all {dropped} agent trajectories exceeded the configured context length; "
                                   f"{self._format_filter_diagnostics(diag)}")
            batch = session.build_train_batch(samples, self.reward_fn)
            self.logger.info("agentic train batch built samples=%d tokens=%d messages=%d tool_calls=%d tool_results=%d",
                             len(samples), sum(len(r) for r in batch.token_rows),
                             sum(len(r.messages) for r in batch.reward_records),
                             sum(len(r.tool_calls) for r in batch.reward_records),
                             sum(len(r.tool_results) for r in batch.reward_records))
            return batch

    @staticmethod
    def _normalize_trajectories(trajectories):
        from ..agentic import AgentTrajectory, AgentTrajectoryTurn

        if isinstance(trajectories, AgentTrajectoryTurn):
            return [[trajectories]]
        if isinstance(trajectories, AgentTrajectory):
            return [trajectories]
        out = []
        for t in trajectories:
            out.append([t] if isinstance(t, AgentTrajectoryTurn) else t)
        return out

    def _context_limit(self, params) -> int | None:
        limits = []
        if getattr(self.config, "max_context_len", None) is not None:
            limits.append(int(self.config.max_context_len))
        try:
            v = self.areno.model_context_len()
        except (AttributeError, RuntimeError):
            v = None
        if v is not None:
            limits.append(int(v))
        return min(limits) if limits else None

    def _filter_overlong(self, samples, params):
        limit = self._context_limit(params)
        if limit is None:
            return samples, 0, {}
        details, kept, dropped = [], [], []
        for s in samples:
            d = {"prompt_idx": s.item.prompt_index, "sample_idx": s.item.sample_index, "tokens": len(s.token_row),
                 "messages": len(s.messages), "assistant_messages": sum(m.get("role") == "assistant" for m in s.messages),
                 "tool_results": sum(m.get("role") == "tool" for m in s.messages),
                 "response_tokens": len(s.response_tokens), "trace_events": len(s.trace),
                 "prompt": str(s.item.prompt).replace("\n", "\\n")[:120]}
            details.append(d)
            (dropped if d["tokens"] > limit else kept).append((s, d))
        lens = sorted(d["tokens"] for d in details)

        def pct(f):
            return int(lens[min(int(round((len(lens) - 1) * f)), len(lens) - 1)]) if lens else 0

        diag = {"max_context_len": limit, "total": len(details), "kept": len(kept), "filtered": len(dropped),
                "min_tokens": lens[0] if lens else 0, "p50_tokens": pct(0.5), "p90_tokens": pct(0.9),
                "max_tokens": lens[-1] if lens else 0,
                "top": sorted((d for _, d in dropped), key=lambda d: d["tokens"], reverse=True)[:5]}
        if dropped:
            self.logger.warning("agentic trajectory filtered: %s", self._format_filter_diagnostics(diag))
        return [s for s, _ in kept], len(dropped), diag

    @staticmethod
    def _format_filter_diagnostics(diag) -> str:
        if not diag:
            return "no context-length diagnostics available"
        top = "; ".join("prompt_idx={prompt_idx} sample_idx={sample_idx} tokens={tokens} messages={messages} "
                        "assistant_messages={assistant_messages} tool_results={tool_results} "
                        "response_tokens={response_tokens} trace_events={trace_events} prompt='{prompt}'".format(**d)
                        for d in diag.get("top", []))
        return ("max_context_len={max_context_len} total={total} kept={kept} filtered={filtered} "
                "tokens[min/p50/p90/max]={min_tokens}/{p50_tokens}/{p90_tokens}/{max_tokens} ").format(**diag) + f"top=[{top}]"

    # --------------------------------------------------------- batch assembly
    def _materialize_train_batch(self, tokenizer, prompt_batch, rollout_results):
        batch, rewards_all, rollout_lp = [], [], []
        eos = getattr(tokenizer, "eos_token_id", None) or 0
        for pi, (item, result) in enumerate(zip(prompt_batch.items, rollout_results)):
            n_p = len(item.input_tokens)
            rewards = []
            for si, seq in enumerate(result.sequences):
                record = make_reward_record(
                    prompt=item.prompt, completion=tokenizer.decode(seq.resp_tokens), source_record=item.record,
                    answer=item.solutions, tokens=item.input_tokens + seq.resp_tokens,
                    logprobs=[0.0] * n_p + seq.resp_logprobs, loss_mask=[False] * n_p + [True] * len(seq.resp_tokens),
                    metadata={"prompt_index": pi, "sample_index": si})
                rewards.append(float(self.reward_fn(record)))
            rewards_all += rewards
            for seq, adv, reward in zip(result.sequences, compute_group_advantages(rewards), rewards):
                n_r = len(seq.resp_tokens)
                rollout_lp += seq.resp_logprobs
                batch.append(TrainSequence(prompt_mask=[True] * n_p + [False] * n_r, tokens=item.input_tokens + seq.resp_tokens,
                                           logprobs=[0.0] * n_p + seq.resp_logprobs, advantages=[0.0] * n_p + [adv] * n_r,
                                           reward=reward, eos_token_id=eos))
        return batch, rewards_all, rollout_lp

    def _materialize_agentic_train_batch(self, tokenizer, prompt_batch, agent_batch):
        if agent_batch.rewards is None:
            raise ValueError("agentic policy training requires a reward_fn")
        rewards = [float(r) for r in agent_batch.rewards]
        groups: dict[int, list[int]] = {}
        for i, rec in enumerate(agent_batch.reward_records):
            groups.setdefault(int(rec.metadata.get("prompt_index", i)), []).append(i)
        adv_by_row: dict[int, float] = {}
        for rows in groups.values():
            for i, a in zip(rows, compute_group_advantages([rewards[i] for i in rows])):
                adv_by_row[i] = float(a)
        batch, rollout_lp = [], []
        eos = getattr(tokenizer, "eos_token_id", None) or 0
        for i, (toks, rmask, lmask, lps, reward) in enumerate(zip(agent_batch.token_rows, agent_batch.response_masks,
                                                                   agent_batch.loss_masks, agent_batch.rollout_logprobs,
                                                                   rewards)):
            if not (len(toks) == len(rmask) == len(lmask) == len(lps)):
                raise ValueError("agentic train batch has misaligned token/mask/logprob rows")
            adv = adv_by_row.get(i, 0.0)
            rollout_lp.extend(lp for lp, on in zip(lps, lmask) if on)
            batch.append(TrainSequence(prompt_mask=[not m for m in rmask], loss_mask=list(lmask), tokens=list(toks),
                                       logprobs=list(lps), advantages=[adv if on else 0.0 for on in lmask],
                                       reward=reward, eos_token_id=eos))
        return batch, rewards, rollout_lp

    # ---------------------------------------------------------------- logging
    def _log_completions(self, tokenizer, epoch, step, prompt_batch, results) -> None:
        limit = int(os.getenv("ARENO_LOG_COMPLETIONS", "0"))
        if limit <= 0:
            return
        n = 0
        for pi, (item, result) in enumerate(zip(prompt_batch.items, results)):
            for si, seq in enumerate(result.sequences):
                self.logger.info("epoch=%d step=%d prompt_idx=%d sample_idx=%d prompt=%r decoded_prompt=%r completion=%r "
                                 "prompt_tokens=%s response_tokens=%s", epoch, step, pi, si, item.prompt,
                                 tokenizer.decode(item.input_tokens), tokenizer.decode(seq.resp_tokens),
                                 item.input_tokens[:64], seq.resp_tokens[:64])
                n += 1
                if n >= limit:
                    return

    def _log_agentic_completions(self, epoch, step, agent_batch) -> None:
        limit = int(os.getenv("ARENO_LOG_COMPLETIONS", "0"))
        for i, rec in enumerate(agent_batch.reward_records[: max(limit, 0)]):
            lmask = agent_batch.loss_masks[i]
            self.logger.info("epoch=%d step=%d prompt_idx=%d sample_idx=%d prompt=%r messages=%s final_answer=%r "
                             "tool_calls=%s tool_results=%s loss_mask_true=%d/%d", epoch, step,
                             int(rec.metadata.get("prompt_index", -1)), int(rec.metadata.get("sample_index", -1)),
                             rec.prompt, rec.messages, rec.final_answer, rec.tool_calls, rec.tool_results[:4],
                             sum(lmask), len(lmask))
