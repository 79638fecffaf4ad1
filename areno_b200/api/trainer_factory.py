"""``build_trainer``: instantiate the trainer class registered for ``config.algo``."""

from __future__ import annotations

from .algorithms import get_algorithm


def build_trainer(config, *, instance, dataset, reward_fn, loss_fn):
    cls = get_algorithm(config.algo).resolve_trainer_cls()
    return cls(config, instance=instance, dataset=dataset, reward_fn=reward_fn, loss_fn=loss_fn)
