"""Prompt containers produced by ``Trainer.load_prompt_batches``."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass
class PromptItem:
    prompt: str
    solutions: list[str] | None
    input_tokens: list[int]
    record: dict[str, Any]


@dataclass
class PromptBatch:
    items: list[PromptItem]
    scanned: int           # raw rows inspected for this batch (including skipped ones)
    skipped_long: int      # rows dropped in this batch for exceeding the prompt budget
    total_skipped_long: int

    @property
    def prompts(self) -> list[str]:
        return [item.prompt for item in self.items]
