"""Typed backend configuration (``areno/api/config.py`` in the reference)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .models import BackendType


@dataclass
class ArenoConfig:
    """Layout and tuning of the native backend.  ``optimizer`` / ``runtime`` are passed verbatim to the
    engine's ``OptimizerConfig`` / ``RuntimeConfig``."""

    model_path: str | None = None       # overrides the Trainer's model path (rarely needed)
    tp_size: int = 1                    # tensor-parallel width of training (and of rollout unless set below)
    dp_size: int | None = None          # None: world_size // tp_size
    # decode tensor-parallel over this many GPUs while training stays data parallel (needs tp_size == 1)
    rollout_tp_size: int | None = None
    # mixture-of-experts models: deal the experts out over the data-parallel ranks and exchange tokens with their
    # owners in every MoE layer, in rollout and training (needs tp_size == 1 and num_experts divisible by the ranks)
    expert_parallel: bool = False
    devices: list[int] | None = None    # GPU ordinals, one per rank; None: 0 .. world_size - 1
    dummy_load: bool = False            # seeded random weights instead of reading the checkpoint
    optimizer: dict[str, Any] = field(default_factory=dict)
    runtime: dict[str, Any] = field(default_factory=dict)
    max_running_prompts: int = 64       # sequences decoded concurrently over the whole job
    decode_progress_interval_s: float = 10.0      # period of the rollout progress log line (0: off)
    # how workers are launched: "spawn" (one process per GPU), "inprocess" (single GPU, no process hop),
    # "spmd" (this process is one of WORLD_SIZE ranks started by torch.distributed.run)
    launcher: str | None = None
    # SPMD launches only (one driver process per rank): every rank hands the Trainer its OWN share of the prompts and
    # training sequences and gets its own results and statistics back; nothing is exchanged between the ranks on
    # the host.  All ranks must make the same calls with the same number of micro-batches.
    spmd_local_data: bool = False
    model_config: Any = None  # explicit ModelConfig (synthetic models without a checkpoint directory)
    seed: int = 0                       # weight initialisation (dummy_load) and the samplers' base seed


BackendConfig = ArenoConfig


def resolve_backend_type(backend_type: BackendType | None, custom_config: Any) -> BackendType:
    del custom_config
    return backend_type if backend_type is not None else BackendType.Areno


def coerce_backend_config(backend_type: BackendType, custom_config: Any) -> BackendConfig | None:
    if custom_config is None:
        return None
    if backend_type == BackendType.Areno and isinstance(custom_config, ArenoConfig):
        return custom_config
    raise TypeError(f"{backend_type.value} requires its typed backend config dataclass, got {type(custom_config)!r}")
