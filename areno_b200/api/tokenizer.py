"""Tokenizer loading and prompt encoding.

Contracts kept from the reference (``areno/api/tokenizer.py:20-133``,
``areno/engine/data/tokenizer.py:14-30``): an optional ``enable_thinking`` switch forwarded to chat
templates that accept it, EOS ids collected from tokenizer + ``config.json`` (top level and
``text_config``), chat template applied unless the prompt already carries chat markers, and token
ids normalised from whatever the tokenizer returns.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

_THINKING_ATTR = "_areno_chat_template_enable_thinking"
_CHAT_MARKERS = ("<|im_start|>", "<start_of_turn>", "<turn|>", "<|user|>", "<|assistant|>")


def load_tokenizer(model_path: str):
    """``AutoTokenizer.from_pretrained`` with a retry for tokenizer configs whose
    ``extra_special_tokens`` is stored as a list (which the stock loader rejects)."""
    from transformers import AutoTokenizer

    try:
        return AutoTokenizer.from_pretrained(model_path, trust_remote_code=True)
    except (AttributeError, TypeError, ValueError):
        cfg_path = Path(model_path) / "tokenizer_config.json"
        if not cfg_path.exists():
            raise
        cfg = json.loads(cfg_path.read_text())
        extra = cfg.get("extra_special_tokens")
        if not isinstance(extra, list):
            raise
        return AutoTokenizer.from_pretrained(model_path, trust_remote_code=True, extra_special_tokens={})


def configure_chat_template_enable_thinking(tokenizer, enable_thinking: bool | None) -> None:
    """``None`` restores the template default; a bool is passed to ``apply_chat_template``."""
    if enable_thinking is None:
        if hasattr(tokenizer, _THINKING_ATTR):
            delattr(tokenizer, _THINKING_ATTR)
        return
    setattr(tokenizer, _THINKING_ATTR, bool(enable_thinking))


def apply_chat_template_with_options(tokenizer, messages, **kwargs):
    kwargs = dict(kwargs)
    thinking = getattr(tokenizer, _THINKING_ATTR, None)
    if thinking is not None:
        kwargs["enable_thinking"] = bool(thinking)
    try:
        return tokenizer.apply_chat_template(messages, **kwargs)
    except TypeError:
        if "enable_thinking" not in kwargs:
            raise
        kwargs.pop("enable_thinking")
        return tokenizer.apply_chat_template(messages, **kwargs)


def _collect(out: list[int], value) -> None:
    if isinstance(value, bool):
        return
    if isinstance(value, int):
        out.append(value)
    elif isinstance(value, (list, tuple)):
        out.extend(v for v in value if isinstance(v, int) and not isinstance(v, bool))


def eos_token_ids(model_path: str | Path, tokenizer) -> tuple[int, ...]:
    ids: list[int] = []
    _collect(ids, getattr(tokenizer, "eos_token_id", None))
    cfg_path = Path(model_path) / "config.json"
    if cfg_path.exists():
        cfg = json.loads(cfg_path.read_text(encoding="utf-8"))
        _collect(ids, cfg.get("eos_token_id"))
        if isinstance(cfg.get("text_config"), dict):
            _collect(ids, cfg["text_config"].get("eos_token_id"))
    return tuple(dict.fromkeys(ids))


def normalize_token_ids(value: Any) -> list[int]:
    """Plain ``list[int]`` from a list, a tokenizers ``Encoding``, a ``BatchEncoding`` or a batch of one."""
    if hasattr(value, "ids"):
        value = value.ids
    if hasattr(value, "input_ids"):
        value = value.input_ids
    if isinstance(value, (list, tuple)):
        if value and hasattr(value[0], "ids"):
            if len(value) != 1:
                raise TypeError("expected one tokenized prompt, got a batch of encodings")
            return normalize_token_ids(value[0])
        if value and isinstance(value[0], (list, tuple)):
            if len(value) != 1:
                raise TypeError("expected one tokenized prompt, got a batch of token id lists")
            return normalize_token_ids(value[0])
        try:
            return [int(t) for t in value]
        except TypeError as exc:
            raise TypeError(f"expected token ids, got {type(value).__name__}") from exc
    if hasattr(value, "tolist"):
        return normalize_token_ids(value.tolist())
    raise TypeError(f"expected token ids or tokenizer Encoding, got {type(value).__name__}")


def looks_chat_formatted(prompt: str) -> bool:
    return any(m in prompt for m in _CHAT_MARKERS)


def encode_generation_prompt(tokenizer, prompt: str) -> list[int]:
    if looks_chat_formatted(prompt) or not getattr(tokenizer, "chat_template", None):
        return normalize_token_ids(tokenizer.encode(prompt))
    return normalize_token_ids(apply_chat_template_with_options(
        tokenizer, [{"role": "user", "content": prompt}], tokenize=True, add_generation_prompt=True))
