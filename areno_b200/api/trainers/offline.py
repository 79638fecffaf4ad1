"""Shared loop of the offline trainers (SFT, DPO): dataset rows -> ``TrainSequence`` batches ->
``Trainer.train``; no rollout, no reward function."""

from __future__ import annotations

import time

from ..tokenizer import configure_chat_template_enable_thinking
from .base import BaseTrainer


class OfflineTrainer(BaseTrainer):
    unit = "rows"

    def _iter_train_batches(self, tokenizer):  # pragma: no cover - abstract
        raise NotImplementedError

    def _prepare(self) -> None:
        pass

    def _before_train(self, train_batch, epoch: int, step: int) -> dict:
        return {}

    def _count(self, train_batch) -> int:
        return len(train_batch)

    def _fit_initialized(self) -> None:
        tokenizer = self.areno.get_tokenizer()
        configure_chat_template_enable_thinking(tokenizer, getattr(self.config, "chat_template_enable_thinking", None))
        self._prepare()
        step = 0
        for epoch in range(self.config.epochs):
            self.logger.info("epoch=%d stage=epoch_start", epoch)
            for batch in self._iter_train_batches(tokenizer):
                if not batch:
                    continue
                extra = self._before_train(batch, epoch, step)
                n = self._count(batch)
                self.logger.info("epoch=%d step=%d role=policy stage=train_start %s=%d", epoch, step, self.unit, n)
                t0 = time.perf_counter()
                result = self.areno.train(batch, self.loss_fn, mini_bs=self.config.mini_bs,
                                          gradient_accumulation_steps=self.config.gradient_accumulation_steps)
                if isinstance(result, dict):
                    result.update(extra)
                    result["policy_train_wall_time_s"] = time.perf_counter() - t0
                self.logger.info("epoch=%d step=%d role=policy stage=train_end %s=%d", epoch, step, self.unit, n)
                self.logger.info("epoch=%d step=%d train_stats=%s", epoch, step, result)
                self._maybe_save(epoch, step)
                step += 1
                if self._reached_max_steps(epoch, step):
                    return
            self.logger.info("epoch=%d stage=epoch_end", epoch)
