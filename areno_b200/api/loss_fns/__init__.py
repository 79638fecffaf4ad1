"""Built-in loss functions; signature ``loss_fn(data_pack, logprobs) -> loss | (loss, metrics)``."""

from .layout import ResponseLayout, masked_mean, response_layout, sequence_sum
from .policy import gspo_loss_fn, grpo_loss_fn, ppo_loss_fn
from .preference import dpo_loss_fn, sft_loss_fn

__all__ = ["ResponseLayout", "masked_mean", "response_layout", "sequence_sum", "gspo_loss_fn", "grpo_loss_fn",
           "ppo_loss_fn", "dpo_loss_fn", "sft_loss_fn"]
