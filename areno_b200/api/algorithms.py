"""Algorithm registry: ``--algo`` names map to a trainer class (loaded lazily), a default loss
function and an optional factory that binds config values into the loss.  Built in: ``sft``,
``dpo``, ``gspo``, ``grpo``, ``ppo``; modules under ``areno_b200.experimental`` register more on
first lookup miss (``areno/api/algorithms.py:25-208`` in the reference)."""

from __future__ import annotations

import importlib
import importlib.util
import pkgutil
from collections.abc import Callable
from dataclasses import dataclass, replace as dc_replace
from functools import partial

from .loss_fns import dpo_loss_fn, grpo_loss_fn, gspo_loss_fn, ppo_loss_fn, sft_loss_fn
from .trainer_config import TrainerConfig

LossFnFactory = Callable[[TrainerConfig, Callable], Callable]


@dataclass(frozen=True)
class AlgorithmSpec:
    name: str
    trainer_cls: type | Callable[[], type]
    default_loss_fn: Callable
    requires_rollout: bool
    loss_fn_factory: LossFnFactory | None = None
    experimental: bool = False

    def resolve_trainer_cls(self) -> type:
        return self.trainer_cls if isinstance(self.trainer_cls, type) else self.trainer_cls()

    def make_loss_fn(self, config: TrainerConfig) -> Callable:
        if self.loss_fn_factory is not None:
            return self.loss_fn_factory(config, self.default_loss_fn)
        return self.default_loss_fn


_ALGORITHMS: dict[str, AlgorithmSpec] = {}
_EXPERIMENTAL_LOADED = False


def register_algorithm(spec: AlgorithmSpec, *, replace: bool = False) -> None:
    name = spec.name.strip().lower()
    if not name:
        raise ValueError("algorithm name must be non-empty")
    if name in _ALGORITHMS and not replace:
        raise ValueError(f"algorithm {name!r} is already registered")
    _ALGORITHMS[name] = spec if name == spec.name else dc_replace(spec, name=name)


def load_experimental_algorithms() -> None:
    """Import every sub-package of ``areno_b200.experimental`` once; each registers its algorithms on import.
    A missing or empty experimental package is not an error."""
    global _EXPERIMENTAL_LOADED
    if _EXPERIMENTAL_LOADED:
        return
    _EXPERIMENTAL_LOADED = True
    root = "areno_b200.experimental"
    if importlib.util.find_spec(root) is None:
        return
    search_path = list(getattr(importlib.import_module(root), "__path__", ()))
    for info in pkgutil.iter_modules(search_path):
        if info.ispkg:
            importlib.import_module(root + "." + info.name)


def get_algorithm(name: str) -> AlgorithmSpec:
    key = name.strip().lower()
    if key not in _ALGORITHMS:
        load_experimental_algorithms()
    if key not in _ALGORITHMS:
        raise ValueError(f"unknown algorithm {name!r}; registered: {', '.join(sorted(_ALGORITHMS))}")
    return _ALGORITHMS[key]


def list_algorithms(*, include_experimental: bool = True) -> dict[str, AlgorithmSpec]:
    if include_experimental:
        load_experimental_algorithms()
    return dict(_ALGORITHMS)


def _policy_trainer() -> type:
    from .trainers.policy_only import PolicyOnlyTrainer

    return PolicyOnlyTrainer


def _sft_trainer() -> type:
    from .trainers.sft import SFTTrainer

    return SFTTrainer


def _dpo_trainer() -> type:
    from .trainers.dpo import DPOTrainer

    return DPOTrainer


def _ppo_trainer() -> type:
    from .trainers.ppo import PPOTrainer

    return PPOTrainer


def _bind_gspo(config, loss_fn):
    return partial(loss_fn, clip_eps=getattr(config, "gspo_clip_eps"))


def _bind_grpo(config, loss_fn):
    return partial(loss_fn, clip_eps=getattr(config, "grpo_clip_eps"))


register_algorithm(AlgorithmSpec("sft", _sft_trainer, sft_loss_fn, requires_rollout=False))
register_algorithm(AlgorithmSpec("dpo", _dpo_trainer, dpo_loss_fn, requires_rollout=False))
register_algorithm(AlgorithmSpec("gspo", _policy_trainer, gspo_loss_fn, requires_rollout=True, loss_fn_factory=_bind_gspo))
register_algorithm(AlgorithmSpec("grpo", _policy_trainer, grpo_loss_fn, requires_rollout=True, loss_fn_factory=_bind_grpo))
register_algorithm(AlgorithmSpec("ppo", _ppo_trainer, ppo_loss_fn, requires_rollout=True))

__all__ = ["AlgorithmSpec", "get_algorithm", "list_algorithms", "load_experimental_algorithms", "register_algorithm"]
