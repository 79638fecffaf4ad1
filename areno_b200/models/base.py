"""Model adapter contract.

An adapter recognises a Hugging Face ``config.json``, derives the normalised ``ModelConfig``,
builds the (tensor-parallel) module on a device and moves weights between the module and HF
safetensors.  Same five-method contract as ``areno/models/base.py:37-70`` in the reference, plus
``init_random`` for seeded synthetic weights.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any

import torch

from ..engine.config import ModelConfig


class ModelAdapter(ABC):
    name: str = ""

    @abstractmethod
    def match_hf_config(self, hf_config: dict[str, Any]) -> bool:
        ...

    @abstractmethod
    def config_from_hf(self, hf_config: dict[str, Any]) -> ModelConfig:
        ...

    @abstractmethod
    def build(self, config: ModelConfig, device: torch.device | str = "cpu") -> torch.nn.Module:
        ...

    @abstractmethod
    def load_weights(self, model: torch.nn.Module, path: str, config: ModelConfig) -> None:
        ...

    @abstractmethod
    def save_weights(self, model: torch.nn.Module, path: str, config: ModelConfig, source_path: str | None = None) -> None:
        ...

    def init_random(self, model: torch.nn.Module, seed: int = 0) -> None:
        from .dense import init_weights

        init_weights(model, seed)
