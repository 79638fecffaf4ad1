"""``Trainer``: the object algorithm scripts talk to.

It owns tokenizer loading, backend construction, step accounting (a step opens at the first
rollout or train call and closes when ``train`` returns), a re-entrant rollout session, the
rollout -> train cycle, role operations for PPO / DPO, checkpointing and optional TensorBoard
recording.  Public methods and their semantics follow ``areno/api/trainer.py:25-425`` of the
reference; ``score_logprobs`` takes its micro-batch size from an attribute of the trainer (the
reference dereferences a non-existent ``self.config`` there).
"""

from __future__ import annotations

import time
from collections.abc import Callable, Iterable
from typing import Any

from .backend.base import Backend, get_backend_cls
from .config import BackendConfig, coerce_backend_config, resolve_backend_type
from .context import Context
from .data import PromptBatch, PromptItem
from .models import BackendType, RolloutResult, SamplingParams, TrainSequence
from .roles import ModelRole
from .tokenizer import encode_generation_prompt, eos_token_ids, load_tokenizer, normalize_token_ids


class Trainer:
    def __init__(self, world_size: int, model_path: str, backend_type: BackendType | None = None,
                 custom_config: BackendConfig | None = None, metrics_log_dir: str | None = None,
                 score_micro_bs: int = 8) -> None:
        self._tokenizer = None
        self._backend: Backend | None = None
        self._backend_type = resolve_backend_type(backend_type, custom_config)
        self._model_path = model_path
        self._ctx: Context | None = None
        self._world_size = world_size
        self._initialized = False
        self._custom_config = coerce_backend_config(self._backend_type, custom_config)
        self._metrics = None
        if metrics_log_dir:
            from .metrics import MetricsRecorder

            self._metrics = MetricsRecorder(metrics_log_dir)
        self._metric_timings: dict[str, float] = {}
        self._step_active = False
        self._step_wall_start: float | None = None
        self._rollout_session_depth = 0
        self._rollout_wall_start: float | None = None
        self.score_micro_bs = int(score_micro_bs)

    # ------------------------------------------------------------- life cycle
    def init(self, tokenizer: Any = None, eos_ids: tuple[int, ...] | None = None) -> None:
        """Load the tokenizer (unless one is supplied), build the context and start the backend."""
        path = self._model_path
        if tokenizer is None and path:
            tokenizer = load_tokenizer(path)
        self._tokenizer = tokenizer
        if eos_ids is None:
            eos_ids = eos_token_ids(path, tokenizer) if path else ()
        self._ctx = Context(self._world_size, path, tokenizer, self._custom_config, tuple(eos_ids))
        if self._backend is None:
            cls = get_backend_cls(self._backend_type)
            if cls is None:
                raise ValueError(f"unsupported backend type: {self._backend_type}")
            self._backend = cls()
        self._backend.initialize(self._ctx)
        self._initialized = True

    @classmethod
    def from_worker(cls, worker, world_size: int = 1, tokenizer: Any = None, eos_ids: tuple[int, ...] = (),
                    max_running_prompts: int | None = None, local_data: bool = False) -> "Trainer":
        """Wrap an already-built rank worker (in-process for one rank, SPMD under torchrun).  ``local_data``: see
        ``ArenoConfig.spmd_local_data``."""
        from ..engine.api import ArenoEngine
        from .backend.native import NativeBackend
        from .config import ArenoConfig

        cfg = ArenoConfig(tp_size=worker.config.tp_size, dp_size=worker.config.dp_size,
                          max_running_prompts=max_running_prompts or worker.config.max_running_seqs * world_size,
                          decode_progress_interval_s=0.0, spmd_local_data=bool(local_data and world_size > 1))
        self = cls(world_size, "", custom_config=cfg)
        launcher = "spmd" if world_size > 1 else "inprocess"
        self._backend = NativeBackend(ArenoEngine(worker.config, launcher=launcher, worker=worker))
        self.init(tokenizer=tokenizer, eos_ids=eos_ids)
        return self

    def get_tokenizer(self) -> Any:
        return self._tokenizer

    def close(self) -> None:
        try:
            if self._backend is not None:
                self._backend.close()
        finally:
            self._backend = None
            self._initialized = False
            if self._metrics is not None:
                self._metrics.close()

    def __enter__(self) -> "Trainer":
        """``with Trainer(...) as trainer:`` initialises on entry (unless ``init`` was called already) and closes on exit."""
        if not self._initialized:
            self.init()
        return self

    def __exit__(self, *_exc) -> None:
        self.close()

    def _require(self) -> tuple[Backend, Context]:
        if self._backend is None or self._ctx is None:
            raise RuntimeError("Trainer is not initialized")
        return self._backend, self._ctx

    # ------------------------------------------------------------------ steps
    def _begin_step(self) -> None:
        _, ctx = self._require()
        if self._step_active:
            return
        ctx.step()
        self._metric_timings = {}
        self._step_active = True
        self._step_wall_start = time.perf_counter()

    def finish_step(self) -> None:
        self._step_active = False
        self._step_wall_start = None

    @property
    def global_step(self) -> int:
        return -1 if self._ctx is None else self._ctx.global_step

    # --------------------------------------------------------------- sessions
    def begin_rollout_session(self) -> None:
        backend, ctx = self._require()
        if self._rollout_session_depth == 0:
            self._begin_step()
            self._rollout_wall_start = time.perf_counter()
            backend.begin_rollout_session(ctx)
        self._rollout_session_depth += 1

    async def begin_rollout_session_async(self) -> None:
        backend, ctx = self._require()
        if self._rollout_session_depth == 0:
            self._begin_step()
            self._rollout_wall_start = time.perf_counter()
            await backend.begin_rollout_session_async(ctx)
        self._rollout_session_depth += 1

    async def sync_rollout_session_async(self) -> None:
        backend, ctx = self._require()
        if self._rollout_session_depth <= 0:
            raise RuntimeError(
                "sync_rollout_session_async must be called inside `async with trainer.rollout_session(...)`")
        await backend.sync_rollout_session_async(ctx)

    def end_rollout_session(self) -> None:
        backend, ctx = self._require()
        if self._rollout_session_depth <= 0:
            return
        self._rollout_session_depth -= 1
        if self._rollout_session_depth == 0:
            try:
                backend.end_rollout_session(ctx)
            finally:
                self._finish_rollout_timing()

    async def end_rollout_session_async(self) -> None:
        backend, ctx = self._require()
        if self._rollout_session_depth <= 0:
            return
        self._rollout_session_depth -= 1
        if self._rollout_session_depth == 0:
            try:
                await backend.end_rollout_session_async(ctx)
            finally:
                self._finish_rollout_timing()

    def _finish_rollout_timing(self) -> None:
        if self._rollout_wall_start is None:
            return
        self._metric_timings["rollout"] = (self._metric_timings.get("rollout", 0.0)
                                           + time.perf_counter() - self._rollout_wall_start)
        self._rollout_wall_start = None

    def rollout_session(self, *, sampling_params: SamplingParams | None = None, loss_mask_policy=None,
                        max_running_prompts: int | None = None, timeout_s: float = 300.0, proxy: bool = True):
        """Session object usable as ``with`` (plain rollouts) or ``async with`` (agentic rollouts behind
        the local OpenAI-compatible proxy)."""
        from .agentic import RolloutSession

        return RolloutSession(self, sampling_params=sampling_params or SamplingParams(),
                              loss_mask_policy=loss_mask_policy, max_running_prompts=max_running_prompts,
                              timeout_s=timeout_s, proxy=proxy)

    # ------------------------------------------------------------------ info
    def dp_size(self) -> int:
        backend, ctx = self._require()
        try:
            return int(backend.dp_size(ctx))
        except AttributeError:
            cfg = ctx.custom_config
            return int(ctx.world_size) if cfg is None else max(int(ctx.world_size) // int(cfg.tp_size), 1)

    def model_context_len(self) -> int | None:
        backend, ctx = self._require()
        return backend.model_context_len(ctx)

    def probe_rollout_cache(self, *, max_new_tokens: int, max_running_prompts: int, max_prompt_len: int) -> float:
        backend, ctx = self._require()
        return backend.probe_rollout_cache(ctx, max_new_tokens=max_new_tokens, max_running_prompts=max_running_prompts,
                                           max_prompt_len=max_prompt_len)

    # ---------------------------------------------------------------- dataset
    def load_prompt_batches(self, dataset, *, batch_size: int, max_prompt_tokens: int, prompt_key: str = "prompt",
                            solutions_key: str = "solutions") -> Iterable[PromptBatch]:
        """Tokenised prompt batches; rows whose prompt exceeds ``max_prompt_tokens`` are skipped (and
        counted), the raw record stays attached for reward functions."""
        cursor = 0
        total_skipped = 0
        n = len(dataset)
        while cursor < n:
            items: list[PromptItem] = []
            scanned = skipped = 0
            while len(items) < batch_size and cursor < n:
                record = dataset[cursor]
                cursor += 1
                scanned += 1
                if prompt_key not in record:
                    raise ValueError(
                        f"dataset row must contain `{prompt_key}`; use --dataset-loader-fn to normalize raw rows")
                prompt = record[prompt_key]
                tokens = encode_generation_prompt(self._tokenizer, prompt)
                if len(tokens) > max_prompt_tokens:
                    skipped += 1
                    total_skipped += 1
                    continue
                items.append(PromptItem(prompt=prompt, solutions=record[solutions_key] if solutions_key in record else None,
                                        input_tokens=tokens, record=dict(record)))
            if not items:
                break
            yield PromptBatch(items=items, scanned=scanned, skipped_long=skipped, total_skipped_long=total_skipped)

    # ---------------------------------------------------------------- rollout
    def rollout_batch(self, prompts: list[str], n_samples: int, sampling_params: SamplingParams) -> list[RolloutResult]:
        tokens = [encode_generation_prompt(self._tokenizer, p) for p in prompts]
        return self.rollout_token_batch(tokens, n_samples, sampling_params)

    def rollout_token_batch(self, prompt_tokens: list[list[int]], n_samples: int,
                            sampling_params: SamplingParams) -> list[RolloutResult]:
        backend, ctx = self._require()
        if self._rollout_session_depth <= 0:
            raise RuntimeError("rollout_token_batch must be called inside `async with trainer.rollout_session(...)`")
        self._begin_step()
        return backend.rollout_batch(ctx, [normalize_token_ids(r) for r in prompt_tokens], n_samples, sampling_params)

    async def rollout_token_batch_async(self, prompt_tokens: list[list[int]], n_samples: int,
                                        sampling_params: SamplingParams) -> list[RolloutResult]:
        backend, ctx = self._require()
        if self._rollout_session_depth <= 0:
            raise RuntimeError(
                "rollout_token_batch_async must be called inside `async with trainer.rollout_session(...)`")
        self._begin_step()
        return await backend.rollout_batch_async(ctx, [normalize_token_ids(r) for r in prompt_tokens], n_samples,
                                                 sampling_params)

    # ------------------------------------------------------------------ train
    def train(self, batch_data: list[TrainSequence], loss_fn: Callable, mini_bs: int = 8,
              gradient_accumulation_steps: int | None = None) -> dict[str, float]:
        if not callable(loss_fn):
            raise TypeError("loss_fn must be callable")
        backend, ctx = self._require()
        self._begin_step()
        start = time.perf_counter()
        result = backend.train(ctx, batch_data, loss_fn, mini_bs, gradient_accumulation_steps)
        self._metric_timings["train"] = time.perf_counter() - start
        if isinstance(result, dict):
            if "rollout" in self._metric_timings:
                result["step_rollout_time_s"] = self._metric_timings["rollout"]
            result["step_train_time_s"] = self._metric_timings["train"]
            if self._step_wall_start is not None:
                result["step_e2e_time_s"] = time.perf_counter() - self._step_wall_start
            from ..utils import tracing

            if tracing.enabled():
                # ARENO_PHASE_TIMERS=1 with an in-process backend: device time of every named phase of this step
                for name, rec in tracing.phase_report().items():
                    result[f"device_ms/{name}"] = rec["ms"]
        if self._metrics is not None:
            self._metrics.record_train_step(step=ctx.global_step, train_result=result, train_batch=batch_data,
                                            timings=self._metric_timings)
        self.finish_step()
        return result

    # ------------------------------------------------------------------ roles
    def ensure_roles(self, roles: dict[str, ModelRole]) -> None:
        backend, ctx = self._require()
        backend.ensure_roles(ctx, roles)

    def score_logprobs(self, role: str, token_rows: list[list[int]]) -> list[list[float]]:
        backend, ctx = self._require()
        return backend.score_logprobs(ctx, role, token_rows, microbatch_size=self.score_micro_bs)

    def score_values(self, role: str, token_rows: list[list[int]]) -> list[list[float]]:
        backend, ctx = self._require()
        return backend.score_values(ctx, role, token_rows)

    def score_rewards(self, role: str, token_rows: list[list[int]]) -> list[float]:
        backend, ctx = self._require()
        return backend.score_rewards(ctx, role, token_rows)

    def train_values(self, role: str, batch_data: list[TrainSequence], mini_bs: int,
                     gradient_accumulation_steps: int | None = None, *, cliprange_value: float = 0.5,
                     value_loss_coef: float = 0.5) -> dict[str, float]:
        backend, ctx = self._require()
        return backend.train_values(ctx, role, batch_data, mini_bs, gradient_accumulation_steps,
                                    cliprange_value=cliprange_value, value_loss_coef=value_loss_coef)

    def save_checkpoint(self, path: str) -> str:
        backend, ctx = self._require()
        return backend.save_checkpoint(ctx, path)
