"""areno_b200: RL post-training on B200 GPUs (sm_100a kernels, paged rollout engine, sharded trainer)."""

import os as _os

__version__ = "0.1.0"

# Training micro-batches are packed to varying token counts, so activation sizes change from one
# micro-batch to the next.  With the caching allocator's fixed-size segments that fragments a nearly
# full device (reserved memory creeps up until cached segments are flushed and re-allocated in the
# middle of a step); expandable segments keep the reservation flat.  A value set by the user wins.
if "PYTORCH_CUDA_ALLOC_CONF" not in _os.environ and "PYTORCH_ALLOC_CONF" not in _os.environ:
    _os.environ["PYTORCH_CUDA_ALLOC_CONF"] = "expandable_segments:True"
    ALLOCATOR_DEFAULT_APPLIED = True
else:
    ALLOCATOR_DEFAULT_APPLIED = False


def configure_allocator() -> None:
    """Apply the allocator default to an already-initialised torch (the environment variable is only
    read when the allocator starts)."""
    if not ALLOCATOR_DEFAULT_APPLIED:
        return
    import torch

    if torch.cuda.is_available():
        try:
            torch.cuda.memory._set_allocator_settings("expandable_segments:True")
        except Exception:  # pragma: no cover - older torch without the setting
            pass


# The names the reference's top-level package offers (``areno/__init__.py:46-66``), resolved on first use so that
# ``import areno_b200`` stays free of torch-heavy imports.
_LAZY_EXPORTS = {
    "ArenoEngine": "areno_b200.engine.api", "EngineConfig": "areno_b200.engine.config",
    "ModelConfig": "areno_b200.engine.config", "OptimizerConfig": "areno_b200.engine.config",
    "RuntimeConfig": "areno_b200.engine.config", "RolloutOutput": "areno_b200.engine.inference",
    "SamplingParams": "areno_b200.engine.inference", "TrainStats": "areno_b200.engine.training",
    "Trainer": "areno_b200.api.trainer",
}


def __getattr__(name: str):
    if name in _LAZY_EXPORTS:
        import importlib

        return getattr(importlib.import_module(_LAZY_EXPORTS[name]), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
