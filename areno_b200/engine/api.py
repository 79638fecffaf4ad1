"""Engine coordinator: the driver-side object that splits work over DP ranks, talks to the worker
cluster and merges results back into caller order.  It holds no weights.

Public surface kept from the reference (``areno/engine/api.py:116-734``): ``from_pretrained``,
``generate_rollout`` / ``generate_rollout_async`` (round-robin DP owner for single requests),
``step``, ``ensure_roles``, ``score_logprobs`` / ``score_values`` / ``score_rewards``,
``train_values``, ``save_checkpoint``, rollout-session begin/sync/end, ``probe_rollout_cache``.
"""

from __future__ import annotations

import itertools
from typing import Any, Callable

import torch

from ..models import registry as model_registry
from .cluster import make_cluster
from .config import EngineConfig, ModelConfig, OptimizerConfig, RuntimeConfig
from .inference import RolloutOutput, SamplingParams
from .protocol import (CachePayload, Op, RolesPayload, RolloutPayload, SavePayload, ScorePayload, TrainPayload,
                       TrainValuesPayload)
from .training import merge_train_stats, split_data_pack_by_dp


def split_list_by_dp(items: list, dp_size: int) -> list[list]:
    return [items[r::dp_size] for r in range(dp_size)]


def dp_rank0_results(results: list, tp_size: int, dp_size: int) -> list:
    """One result per DP row: the one reported by its TP rank 0."""
    return [results[d * tp_size] for d in range(dp_size)]


# statistics of a rollout that describe the slowest rank rather than a total
_STATS_MAX_OVER_RANKS = ("decode_steps", "wall_s")


def merge_rollouts_in_input_order(outputs: list[RolloutOutput], total: int) -> RolloutOutput:
    """One output for ``total`` prompts from the ranks' shares (each names the input positions of its rows).  Numeric
    statistics are summed over the ranks, except the ones that every rank measures for the same loop (steps, wall
    time), which take the largest value."""
    merged = RolloutOutput(tokens=[[] for _ in range(total)], logprobs=[[] for _ in range(total)],
                           finish_reasons=["" for _ in range(total)], prompt_indices=list(range(total)))
    for out in outputs:
        if out is None:
            continue
        for j, idx in enumerate(out.prompt_indices or []):
            merged.tokens[idx] = out.tokens[j]
            merged.logprobs[idx] = out.logprobs[j]
            merged.finish_reasons[idx] = out.finish_reasons[j]
        for key, val in (out.stats or {}).items():
            if not isinstance(val, (int, float)) or isinstance(val, bool):
                merged.stats.setdefault(key, val)
            elif key in _STATS_MAX_OVER_RANKS:
                merged.stats[key] = max(merged.stats.get(key, val), val)
            else:
                merged.stats[key] = merged.stats.get(key, 0) + val
    return merged


class ArenoEngine:
    def __init__(self, config: EngineConfig, loss_fn: Callable | None = None, launcher: str | None = None,
                 worker=None):
        self.loss_fn = loss_fn if loss_fn is not None else config.train_loss_fn
        if config.train_loss_fn is not None:
            # the loss travels with the packs; the copy of the configuration that goes to the workers carries none
            # (it is pickled for spawned workers, which a closure would not survive)
            import copy

            config = copy.copy(config)
            config.train_loss_fn = None
        self.config = config
        self.cluster = make_cluster(config, launcher, worker)
        self._dp_cursor = itertools.count()

    @classmethod
    def from_pretrained(cls, model: str | None, *, tp_size: int = 1, dp_size: int | None = None,
                        devices: list[int] | None = None, dummy_load: bool = False,
                        optimizer_config: OptimizerConfig | None = None, runtime_config: RuntimeConfig | None = None,
                        loss_fn: Callable | None = None, model_config: ModelConfig | None = None,
                        launcher: str | None = None, max_running_seqs: int = 64, seed: int = 0,
                        backend: str | None = None, rollout_tp_size: int | None = None,
                        expert_parallel: bool = False) -> "ArenoEngine":
        if model_config is None:
            if model is None:
                raise ValueError("from_pretrained() requires a local model path or an explicit model_config")
            from ..cli.model_refs import resolve_model_path

            model = resolve_model_path(model)
            _adapter, model_config = model_registry.config_from_pretrained(model)
        cfg = EngineConfig(model=model_config, model_path=model or "", tp_size=tp_size, dp_size=dp_size, devices=devices,
                           dummy_load=dummy_load or not model, optimizer=optimizer_config or OptimizerConfig(),
                           runtime=runtime_config or RuntimeConfig(), max_running_seqs=max_running_seqs, seed=seed,
                           backend=backend, rollout_tp_size=rollout_tp_size, expert_parallel=expert_parallel)
        return cls(cfg, loss_fn=loss_fn, launcher=launcher)

    # ---------------------------------------------------------------- sessions
    def begin_rollout_session(self) -> None:
        self.cluster.call(Op.ROLLOUT_SESSION_BEGIN)

    async def begin_rollout_session_async(self) -> None:
        await self.cluster.call_async(Op.ROLLOUT_SESSION_BEGIN)

    async def sync_rollout_session_async(self) -> None:
        await self.cluster.call_async(Op.ROLLOUT_SESSION_SYNC)

    def end_rollout_session(self) -> None:
        self.cluster.call(Op.ROLLOUT_SESSION_END)

    async def end_rollout_session_async(self) -> None:
        await self.cluster.call_async(Op.ROLLOUT_SESSION_END)

    # ----------------------------------------------------------------- rollout
    def _rollout_payload(self, prompts, indices_by_dp, prompts_by_dp, *, max_new_tokens, max_running_prompts,
                         eos_token_id, sampling_params, decode_progress_interval_s, cancel_flags) -> RolloutPayload:
        dp = int(self.config.rollout_dp)
        if eos_token_id is None:
            eos = ()
        elif isinstance(eos_token_id, int):
            eos = (eos_token_id,)
        else:
            eos = tuple(int(t) for t in eos_token_id)
        local_running = max((max_running_prompts + dp - 1) // dp, 1)
        max_cache_len = max(len(p) for p in prompts) + max_new_tokens
        return RolloutPayload(prompts_by_dp=prompts_by_dp, prompt_indices_by_dp=indices_by_dp,
                              max_new_tokens=max_new_tokens, eos_token_ids=eos,
                              sampling_params=sampling_params or SamplingParams(), max_running_seqs=local_running,
                              max_cache_len=max_cache_len, decode_progress_interval_s=decode_progress_interval_s,
                              cancel_flags=cancel_flags)

    def generate_rollout(self, prompts: list[list[int]], *, max_new_tokens: int, max_running_prompts: int,
                         max_prompt_len: int | None = None, eos_token_id=None,
                         sampling_params: SamplingParams | None = None, decode_progress_interval_s: float = 0.0,
                         cancel_flags: torch.Tensor | None = None, local: bool = False) -> RolloutOutput:
        """One completion per prompt, merged over DP ranks in input order.  ``local`` (SPMD launches): ``prompts``
        are this rank's own share, generated by its own data-parallel row and returned to it alone."""
        if local:
            return self._generate_rollout_local(prompts, max_new_tokens=max_new_tokens,
                                                max_running_prompts=max_running_prompts, eos_token_id=eos_token_id,
                                                sampling_params=sampling_params,
                                                decode_progress_interval_s=decode_progress_interval_s,
                                                cancel_flags=cancel_flags)
        if not prompts:
            raise ValueError("prompts must be non-empty")
        if max_running_prompts < 1:
            raise ValueError("max_running_prompts must be >= 1")
        dp = int(self.config.rollout_dp)
        payload = self._rollout_payload(
            prompts, split_list_by_dp(list(range(len(prompts))), dp), split_list_by_dp(prompts, dp),
            max_new_tokens=max_new_tokens, max_running_prompts=max_running_prompts, eos_token_id=eos_token_id,
            sampling_params=sampling_params, decode_progress_interval_s=decode_progress_interval_s,
            cancel_flags=cancel_flags)
        results = self.cluster.call(Op.INFER_ROLLOUT, payload)
        return merge_rollouts_in_input_order(dp_rank0_results(results, self.config.rollout_tp, dp), len(prompts))

    def _require_spmd(self):
        if not getattr(self.cluster, "is_spmd", False):
            raise RuntimeError("rank-local data needs the SPMD launcher (one driver process per rank, e.g. torchrun)")
        return self.cluster.worker

    def _generate_rollout_local(self, prompts, *, max_new_tokens, max_running_prompts, eos_token_id, sampling_params,
                                decode_progress_interval_s, cancel_flags) -> RolloutOutput:
        worker = self._require_spmd()
        dp, mine = int(self.config.rollout_dp), int(worker.rollout_ctx.dp_rank)
        prompts = list(prompts)
        if sampling_params is not None and sampling_params.seed is not None:
            # every row numbers its own prompts from zero: keep the rows' seeded streams apart
            from dataclasses import replace

            sampling_params = replace(sampling_params, seed=(int(sampling_params.seed) + 0x9E3779B1 * mine) & 0x7FFFFFFF)
        by_dp = [prompts if r == mine else [] for r in range(dp)]
        idx_by_dp = [list(range(len(prompts))) if r == mine else [] for r in range(dp)]
        payload = self._rollout_payload(prompts or [[0]], idx_by_dp, by_dp, max_new_tokens=max_new_tokens,
                                        max_running_prompts=max_running_prompts, eos_token_id=eos_token_id,
                                        sampling_params=sampling_params,
                                        decode_progress_interval_s=decode_progress_interval_s, cancel_flags=cancel_flags)
        results = self.cluster.call(Op.INFER_ROLLOUT, payload, gather=False)
        return merge_rollouts_in_input_order(results, len(prompts))

    async def generate_rollout_async(self, prompts: list[list[int]], *, max_new_tokens: int, max_running_prompts: int,
                                     max_prompt_len: int | None = None, eos_token_id=None,
                                     sampling_params: SamplingParams | None = None,
                                     decode_progress_interval_s: float = 0.0,
                                     cancel_flags: torch.Tensor | None = None) -> RolloutOutput:
        """Request-concurrent rollout: the whole request goes to one DP row chosen round-robin, where it
        joins that worker's running batch; only that row's TP-rank-0 result is awaited."""
        if not prompts:
            raise ValueError("prompts must be non-empty")
        if self.config.expert_parallel:
            raise RuntimeError("request-concurrent rollout sends a request to one data-parallel row; with expert "
                               "parallelism every rank takes part in every forward pass: use generate_rollout")
        dp, tp = int(self.config.rollout_dp), int(self.config.rollout_tp)
        owner = next(self._dp_cursor) % dp
        prompts_by_dp = [[] for _ in range(dp)]
        indices_by_dp = [[] for _ in range(dp)]
        prompts_by_dp[owner] = list(prompts)
        indices_by_dp[owner] = list(range(len(prompts)))
        payload = self._rollout_payload(
            prompts, indices_by_dp, prompts_by_dp, max_new_tokens=max_new_tokens,
            max_running_prompts=max_running_prompts * dp, eos_token_id=eos_token_id, sampling_params=sampling_params,
            decode_progress_interval_s=decode_progress_interval_s, cancel_flags=cancel_flags)
        results = await self.cluster.call_async(Op.INFER_ROLLOUT, payload, result_ranks={owner * tp})
        picked = [r for r in results if isinstance(r, RolloutOutput) and r.prompt_indices]
        return merge_rollouts_in_input_order(picked, len(prompts))

    def probe_rollout_cache(self, *, max_new_tokens: int, max_running_prompts: int, max_prompt_len: int) -> float:
        if min(max_running_prompts, max_prompt_len, max_new_tokens) < 1:
            raise ValueError("max_running_prompts, max_prompt_len and max_new_tokens must be >= 1")
        dp = int(self.config.rollout_dp)
        res = self.cluster.call(Op.PROBE_ROLLOUT_CACHE, CachePayload(max((max_running_prompts + dp - 1) // dp, 1),
                                                                     max_prompt_len + max_new_tokens))
        return max(float(r or 0.0) for r in res) if res else 0.0

    # ------------------------------------------------------------------- train
    def step(self, data_packs: list[dict[str, Any]], *, gradient_accumulation_steps: int | None = None,
             local: bool = False) -> list[dict]:
        """``local`` (SPMD launches): ``data_packs`` hold this rank's own sequences; every rank must pass the same
        number of packs.  The returned statistics are this rank's own."""
        if not data_packs:
            return []
        if self.loss_fn is not None:
            for p in data_packs:          # packs may bring their own loss; the engine's is the default
                if isinstance(p, dict):
                    p.setdefault("_loss_fn", self.loss_fn)
        dp = int(self.config.dp_size)
        if local:
            worker = self._require_spmd()
            from ..parallel.context import get_context

            mine = int(get_context().dp_rank)
            del worker
            packs_by_dp = [[p if r == mine else None for r in range(dp)] for p in data_packs]
            results = self.cluster.call(Op.TRAIN, TrainPayload(packs_by_dp, gradient_accumulation_steps), gather=False)
            return [merge_train_stats([st]) for st in results[0]]
        packs_by_dp = [split_data_pack_by_dp(p, dp) for p in data_packs]
        results = self.cluster.call(Op.TRAIN, TrainPayload(packs_by_dp, gradient_accumulation_steps))
        stats = []
        for per_step in zip(*results):
            stats.append(merge_train_stats(dp_rank0_results(list(per_step), self.config.tp_size, dp)))
        return stats

    # ------------------------------------------------------------------- roles
    def ensure_roles(self, roles: dict[str, Any]) -> None:
        self.cluster.call(Op.ENSURE_ROLES, RolesPayload(roles))

    def _score(self, op: Op, role: str, rows: list[list[int]], pad_token_id: int, microbatch_size: int = 8) -> list:
        dp = int(self.config.dp_size)
        results = self.cluster.call(op, ScorePayload(role, split_list_by_dp(rows, dp), pad_token_id, microbatch_size))
        per_dp = dp_rank0_results(results, self.config.tp_size, dp)
        out: list = [None] * len(rows)
        for r, vals in enumerate(per_dp):
            for j, v in enumerate(vals or []):
                out[r + j * dp] = v
        return out

    def score_logprobs(self, role, token_rows, *, pad_token_id: int = 0, microbatch_size: int = 8):
        return self._score(Op.SCORE_LOGPROBS, role, token_rows, pad_token_id, microbatch_size)

    def score_values(self, role, token_rows, *, pad_token_id: int = 0):
        return self._score(Op.SCORE_VALUES, role, token_rows, pad_token_id)

    def score_rewards(self, role, token_rows, *, pad_token_id: int = 0):
        return self._score(Op.SCORE_REWARDS, role, token_rows, pad_token_id)

    def train_values(self, role, data_packs, *, gradient_accumulation_steps=None, cliprange_value=0.5,
                     value_loss_coef=0.5):
        dp = int(self.config.dp_size)
        packs_by_dp = [split_data_pack_by_dp(p, dp) for p in data_packs]
        results = self.cluster.call(Op.TRAIN_VALUES, TrainValuesPayload(role, packs_by_dp, gradient_accumulation_steps,
                                                                       cliprange_value, value_loss_coef))
        # every rank answers with one flat dict of critic statistics for the whole call: mean over the DP replicas
        per_dp = [r for r in dp_rank0_results(list(results), self.config.tp_size, dp) if r]
        if not per_dp:
            return {}
        return {k: sum(float(r[k]) for r in per_dp if k in r) / sum(1 for r in per_dp if k in r) for k in per_dp[0]}

    # -------------------------------------------------------------------- misc
    def save_checkpoint(self, path: str) -> str:
        self.cluster.call(Op.SAVE_CHECKPOINT, SavePayload(path))
        return path

    def model_info(self) -> dict:
        return self.cluster.call(Op.MODEL_INFO)[0]

    def close(self) -> None:
        self.cluster.close()

    def __enter__(self) -> "ArenoEngine":
        return self

    def __exit__(self, *_exc) -> None:
        self.close()
