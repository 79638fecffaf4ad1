"""Import path of the reference (``areno/api/loss_fns/ppo.py``); the loss lives in ``policy.py`` with the other policy losses."""

from .policy import ppo_loss_fn

__all__ = ["ppo_loss_fn"]
