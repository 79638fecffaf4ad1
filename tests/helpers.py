"""Shared test fixtures: a tiny dense model config, a whitespace tokenizer, a saved checkpoint dir."""

from __future__ import annotations

import json
import os

import torch

from areno_b200.engine.config import ModelConfig


def tiny_config(**kw) -> ModelConfig:
    base = dict(model_type="qwen2", vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, head_dim=32, rope_theta=1e4, qk_norm=False,
                qkv_bias=True, dtype=torch.float32, max_position_embeddings=512)
    base.update(kw)
    return ModelConfig(**base)


class FakeTokenizer:
    """Deterministic word-hash tokenizer with the attributes the SDK reads."""

    chat_template = None
    pad_token_id = 0
    bos_token_id = 1
    eos_token_id = 2
    unk_token_id = None
    all_special_ids = [0, 1, 2]
    name_or_path = "fake"

    def __init__(self, vocab_size: int = 512):
        self.vocab_size = vocab_size
        self._words: dict[int, str] = {}

    def encode(self, text: str, add_special_tokens: bool = True):
        ids = []
        for w in str(text).split():
            t = 3 + (sum(ord(c) * (i + 1) for i, c in enumerate(w)) % (self.vocab_size - 3))
            self._words.setdefault(t, w)
            ids.append(t)
        return ids or [3]

    def decode(self, ids, skip_special_tokens: bool = True):
        return " ".join(self._words.get(int(t), f"<{int(t)}>") for t in ids
                        if not (skip_special_tokens and int(t) in self.all_special_ids))


def write_tiny_checkpoint(path: str, seed: int = 0, **kw) -> ModelConfig:
    """Build the tiny model with seeded random weights and save it as an HF safetensors directory."""
    from areno_b200.engine.checkpoint import save_dense_checkpoint
    from areno_b200.models.dense import DenseCausalLM, init_weights
    from areno_b200.parallel.context import single_process_context

    single_process_context()
    cfg = tiny_config(**kw)
    model = DenseCausalLM(cfg)
    init_weights(model, seed)
    save_dense_checkpoint(model, path, cfg)
    hf = json.load(open(os.path.join(path, "config.json")))
    hf["eos_token_id"] = 2
    json.dump(hf, open(os.path.join(path, "config.json"), "w"))
    return cfg
