"""Per-trainer runtime context handed to every backend call."""

from __future__ import annotations

from .config import BackendConfig


class Context:
    def __init__(self, world_size, model_path: str, tokenizer, custom_config: BackendConfig | None = None,
                 eos_token_ids: tuple[int, ...] = ()):
        self.model_path = model_path
        self.world_size = world_size
        self.global_step = -1  # the first opened step is step 0
        self.tokenizer = tokenizer
        self.custom_config = custom_config
        self.eos_token_ids = eos_token_ids

    def step(self) -> int:
        self.global_step += 1
        return self.global_step
