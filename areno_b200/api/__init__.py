"""Public SDK surface (lazy).  Names mirror ``areno/api/__init__.py:37-66`` of the reference."""

from __future__ import annotations

import importlib

_EXPORTS = {
    "Trainer": "areno_b200.api.trainer",
    "AlgorithmSpec": "areno_b200.api.algorithms",
    "get_algorithm": "areno_b200.api.algorithms",
    "list_algorithms": "areno_b200.api.algorithms",
    "register_algorithm": "areno_b200.api.algorithms",
    "ArenoConfig": "areno_b200.api.config",
    "PromptBatch": "areno_b200.api.data",
    "PromptItem": "areno_b200.api.data",
    "AgentBatch": "areno_b200.api.agentic",
    "AgentItem": "areno_b200.api.agentic",
    "AgentTrainBatch": "areno_b200.api.agentic",
    "AgentTrajectory": "areno_b200.api.agentic",
    "AgentTrajectoryTurn": "areno_b200.api.agentic",
    "LossMaskPolicy": "areno_b200.api.agentic",
    "RolloutSession": "areno_b200.api.agentic",
    "RewardEvent": "areno_b200.api.rewards",
    "RewardRecord": "areno_b200.api.rewards",
    "SamplingParams": "areno_b200.api.models",
    "RolloutResult": "areno_b200.api.models",
    "RolloutSequence": "areno_b200.api.models",
    "TrainSequence": "areno_b200.api.models",
    "BackendType": "areno_b200.api.models",
    "dpo_loss_fn": "areno_b200.api.loss_fns",
    "gspo_loss_fn": "areno_b200.api.loss_fns",
    "grpo_loss_fn": "areno_b200.api.loss_fns",
    "ppo_loss_fn": "areno_b200.api.loss_fns",
    "sft_loss_fn": "areno_b200.api.loss_fns",
}
def __getattr__(name: str):
    if name in ("Areno", "DefaultBackend"):     # the backend selector, as in ``areno/api/__init__.py:34-35``
        return importlib.import_module("areno_b200.api.models").BackendType.Areno
    if name in _EXPORTS:
        return getattr(importlib.import_module(_EXPORTS[name]), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = list(_EXPORTS) + ["Areno", "DefaultBackend"]
