"""Import path of the reference (``areno/api/loss_fns/grpo.py``); the loss lives in ``policy.py`` with the other policy losses."""

from .policy import grpo_loss_fn

__all__ = ["grpo_loss_fn"]
