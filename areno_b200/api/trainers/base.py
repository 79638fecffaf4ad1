"""Shared skeleton of the algorithm trainers: the epoch / step loop, structured ``key=value`` stage
logs, save cadence (``save_path/step_{n:06d}`` every ``save_interval`` steps) and stop conditions."""

from __future__ import annotations

import os

from ...utils.log import get_logger


class BaseTrainer:
    def __init__(self, config, *, instance, dataset, reward_fn=None, loss_fn=None):
        self.config = config
        self.areno = instance
        self.dataset = dataset
        self.reward_fn = reward_fn
        self.loss_fn = loss_fn
        self.logger = get_logger(type(self).__name__)

    def fit(self) -> None:
        self.areno.init()
        try:
            self._fit_initialized()
        finally:
            self.areno.close()

    def _fit_initialized(self) -> None:  # pragma: no cover - abstract
        raise NotImplementedError

    def _reached_max_steps(self, epoch: int, step: int) -> bool:
        if self.config.max_steps is not None and step >= self.config.max_steps:
            self.logger.info("epoch=%d step=%d stage=max_steps_reached", epoch, step)
            return True
        return False

    def _maybe_save(self, epoch: int, step: int) -> None:
        path, every = self.config.save_path, int(self.config.save_interval or 0)
        if not path or every <= 0 or (step + 1) % every != 0:
            return
        target = os.path.join(path, f"step_{step + 1:06d}")
        self.logger.info("epoch=%d step=%d stage=save_start path=%s", epoch, step, target)
        self.areno.save_checkpoint(target)
        self.logger.info("epoch=%d step=%d stage=save_end path=%s", epoch, step, target)
