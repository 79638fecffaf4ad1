"""Import path of the reference (``areno/api/loss_fns/dpo.py``); the loss lives in ``preference.py``."""

from .preference import dpo_loss_fn

__all__ = ["dpo_loss_fn"]
