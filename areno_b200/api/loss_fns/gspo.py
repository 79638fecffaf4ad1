"""Import path of the reference (``areno/api/loss_fns/gspo.py``); the loss lives in ``policy.py`` with the other policy losses."""

from .policy import gspo_loss_fn

__all__ = ["gspo_loss_fn"]
