"""Adapters for the dense pre-norm decoder families: Llama, Qwen2 / Qwen2.5, Qwen3.

The reference covers Llama and Qwen3 (``areno/models/llama/model.py:28-70``,
``areno/models/qwen3/model.py:394-440``) and runs Qwen2.5-shaped models only by relabelling their
config as ``qwen3``; here ``qwen2`` is matched directly (attention bias on, no q/k norm).
"""

from __future__ import annotations

from typing import Any


from ..engine.config import ModelConfig, parse_dtype
from .base import ModelAdapter
from .dense import DenseCausalLM

def _common(hf: dict[str, Any], **over) -> ModelConfig:
    heads = int(hf["num_attention_heads"])
    hidden = int(hf["hidden_size"])
    cfg = dict(
        model_type=hf.get("model_type", "llama"),
        vocab_size=int(hf["vocab_size"]),
        hidden_size=hidden,
        intermediate_size=int(hf.get("intermediate_size", 4 * hidden)),
        num_hidden_layers=int(hf["num_hidden_layers"]),
        num_attention_heads=heads,
        num_key_value_heads=int(hf.get("num_key_value_heads") or heads),
        head_dim=int(hf.get("head_dim") or hidden // heads),
        rms_norm_eps=float(hf.get("rms_norm_eps", 1e-6)),
        rope_theta=float(hf.get("rope_theta") or (hf.get("rope_parameters") or {}).get("rope_theta", 10000.0)),
        max_position_embeddings=int(hf.get("max_position_embeddings", 4096)),
        tie_word_embeddings=bool(hf.get("tie_word_embeddings", False)),
        hidden_act=hf.get("hidden_act", "silu"),
        dtype=parse_dtype(hf.get("torch_dtype") or hf.get("dtype")),
    )
    cfg.update(over)
    return ModelConfig(**cfg)


class _DenseAdapter(ModelAdapter):
    model_types: tuple[str, ...] = ()

    def match_hf_config(self, hf_config):
        return hf_config.get("model_type") in self.model_types

    def build(self, config, device="cpu"):
        return DenseCausalLM(config, device=device)

    def load_weights(self, model, path, config):
        from ..engine.checkpoint import load_dense_checkpoint

        load_dense_checkpoint(model, path, config)

    def save_weights(self, model, path, config, source_path=None):
        from ..engine.checkpoint import save_dense_checkpoint

        save_dense_checkpoint(model, path, config, source_path)


class LlamaAdapter(_DenseAdapter):
    name = "llama"
    model_types = ("llama",)

    def config_from_hf(self, hf):
        return _common(hf, model_type="llama", qk_norm=False, qkv_bias=bool(hf.get("attention_bias", False)),
                       use_bias=bool(hf.get("mlp_bias", False)))


class Qwen2Adapter(_DenseAdapter):
    name = "qwen2"
    model_types = ("qwen2",)

    def config_from_hf(self, hf):
        return _common(hf, model_type="qwen2", qk_norm=False, qkv_bias=True,
                       rope_theta=float(hf.get("rope_theta", 1_000_000.0)))


class Qwen3Adapter(_DenseAdapter):
    name = "qwen3"
    model_types = ("qwen3",)

    def config_from_hf(self, hf):
        return _common(hf, model_type="qwen3", qk_norm=bool(hf.get("qk_layernorm", True)),
                       qkv_bias=bool(hf.get("attention_bias", False)),
                       rope_theta=float(hf.get("rope_theta", 1_000_000.0)))


ADAPTERS = [LlamaAdapter, Qwen2Adapter, Qwen3Adapter]
