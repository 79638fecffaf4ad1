"""Import path of the reference (``areno/api/loss_fns/sft.py``); the loss lives in ``preference.py``."""

from .preference import sft_loss_fn

__all__ = ["sft_loss_fn"]
