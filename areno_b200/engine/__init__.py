"""Engine layer.  Heavy modules are imported lazily so ``import areno_b200.engine`` stays cheap."""

from __future__ import annotations

_LAZY = {
    "ArenoEngine": ("areno_b200.engine.api", "ArenoEngine"),
    "EngineConfig": ("areno_b200.engine.config", "EngineConfig"),
    "ModelConfig": ("areno_b200.engine.config", "ModelConfig"),
    "OptimizerConfig": ("areno_b200.engine.config", "OptimizerConfig"),
    "RuntimeConfig": ("areno_b200.engine.config", "RuntimeConfig"),
    "SamplingParams": ("areno_b200.engine.inference", "SamplingParams"),
    "RolloutOutput": ("areno_b200.engine.inference", "RolloutOutput"),
    "TrainStats": ("areno_b200.engine.training", "TrainStats"),
}


def __getattr__(name: str):
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = list(_LAZY)
