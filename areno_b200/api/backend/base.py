"""Backend boundary: what the SDK needs from an execution engine.

``initialize / rollout_batch / train`` are required; everything else has a default that either
does nothing or raises ``MissingRoleCapability``.  Backends register by ``BackendType`` and are
imported lazily (``areno/api/backend/base.py:18-187`` in the reference).
"""

from __future__ import annotations

import importlib
from abc import ABC, abstractmethod
from typing import Any, Callable

from ..context import Context
from ..models import BackendType, RolloutResult, SamplingParams, TrainSequence
from ..roles import MissingRoleCapability, ModelRole

_BACKENDS: dict[BackendType, type] = {}
_LAZY_MODULES: dict[BackendType, str] = {BackendType.Areno: "areno_b200.api.backend.native"}


def register_backend(backend_type: BackendType):
    def deco(cls):
        _BACKENDS[backend_type] = cls
        return cls

    return deco


def get_backend_cls(backend_type: BackendType):
    if backend_type not in _BACKENDS and backend_type in _LAZY_MODULES:
        importlib.import_module(_LAZY_MODULES[backend_type])
    return _BACKENDS.get(backend_type)


class Backend(ABC):
    def __init__(self) -> None:
        pass

    @abstractmethod
    def initialize(self, ctx: Context) -> None:
        ...

    @abstractmethod
    def rollout_batch(self, ctx: Context, prompt_tokens: list[list[int]], n_samples: int,
                      sampling_params: SamplingParams) -> list[RolloutResult]:
        ...

    @abstractmethod
    def train(self, ctx: Context, batch_data: list[TrainSequence], loss_fn: Callable, mini_bs: int,
              gradient_accumulation_steps: int | None = None) -> dict[str, Any]:
        ...

    async def rollout_batch_async(self, ctx, prompt_tokens, n_samples, sampling_params):
        return self.rollout_batch(ctx, prompt_tokens, n_samples, sampling_params)

    def begin_rollout_session(self, ctx: Context) -> None:
        pass

    async def begin_rollout_session_async(self, ctx: Context) -> None:
        self.begin_rollout_session(ctx)

    async def sync_rollout_session_async(self, ctx: Context) -> None:
        pass

    def end_rollout_session(self, ctx: Context) -> None:
        pass

    async def end_rollout_session_async(self, ctx: Context) -> None:
        self.end_rollout_session(ctx)

    def dp_size(self, ctx: Context) -> int:
        cfg = ctx.custom_config
        tp = int(getattr(cfg, "tp_size", 1) or 1)
        return max(int(ctx.world_size) // tp, 1)

    def model_context_len(self, ctx: Context) -> int | None:
        return None

    def probe_rollout_cache(self, ctx: Context, *, max_new_tokens: int, max_running_prompts: int,
                            max_prompt_len: int) -> float:
        return 0.0

    def save_checkpoint(self, ctx: Context, path: str) -> str:
        raise MissingRoleCapability(f"{type(self).__name__} cannot save checkpoints")

    def ensure_roles(self, ctx: Context, roles: dict[str, ModelRole]) -> None:
        raise MissingRoleCapability(f"{type(self).__name__} does not support model roles")

    def score_logprobs(self, ctx, role, token_rows, *, microbatch_size: int = 8):
        raise MissingRoleCapability(f"{type(self).__name__} cannot score logprobs")

    def score_values(self, ctx, role, token_rows):
        raise MissingRoleCapability(f"{type(self).__name__} cannot score values")

    def score_rewards(self, ctx, role, token_rows):
        raise MissingRoleCapability(f"{type(self).__name__} cannot score rewards")

    def train_values(self, ctx, role, batch_data, mini_bs, gradient_accumulation_steps=None, *,
                     cliprange_value: float = 0.5, value_loss_coef: float = 0.5):
        raise MissingRoleCapability(f"{type(self).__name__} cannot train value roles")

    def close(self) -> None:
        pass
