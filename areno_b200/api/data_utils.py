"""Dataset tokenisation helpers shared by the offline trainers (SFT / DPO)."""

from __future__ import annotations

from typing import Any

from .tokenizer import apply_chat_template_with_options, encode_generation_prompt, normalize_token_ids


def _flatten_messages(messages: list[dict[str, Any]]) -> str:
    return "\n".join(f"{m.get('role', 'user')}: {m.get('content', '')}" for m in messages)


def apply_chat_template(tokenizer, messages: list[dict[str, Any]]) -> list[int]:
    """Full conversation -> ids (no generation prompt); plain ``role: content`` lines for base tokenizers."""
    if getattr(tokenizer, "chat_template", None):
        return normalize_token_ids(apply_chat_template_with_options(tokenizer, messages, tokenize=True,
                                                                    add_generation_prompt=False))
    return normalize_token_ids(tokenizer.encode(_flatten_messages(messages), add_special_tokens=False))


def encode_prompt_value(tokenizer, prompt) -> list[int]:
    """A preference prompt may be text or a list of chat messages."""
    if isinstance(prompt, list):
        if getattr(tokenizer, "chat_template", None):
            return normalize_token_ids(apply_chat_template_with_options(tokenizer, prompt, tokenize=True,
                                                                        add_generation_prompt=True))
        return encode_generation_prompt(tokenizer, _flatten_messages(prompt))
    return encode_generation_prompt(tokenizer, prompt)


def response_to_tokens_and_mask(prompt_ids: list[int], response: str, tokenizer, eos_token_id: int | None):
    resp = normalize_token_ids(tokenizer.encode(response, add_special_tokens=False))
    if eos_token_id is not None and (not resp or resp[-1] != eos_token_id):
        resp.append(eos_token_id)
    return prompt_ids + resp, [True] * len(prompt_ids) + [False] * len(resp)


def prompt_response_to_tokens_and_mask(prompt: str, response: str, tokenizer, eos_token_id: int | None):
    return response_to_tokens_and_mask(encode_generation_prompt(tokenizer, prompt), response, tokenizer, eos_token_id)


def has_any(record: dict[str, Any], keys: tuple[str, ...]) -> bool:
    return any(isinstance(record.get(k), str) for k in keys)


def first_text(record: dict[str, Any], keys: tuple[str, ...]) -> str:
    for k in keys:
        if isinstance(record.get(k), str):
            return record[k]
    raise KeyError(keys[0])


def first_value(record: dict[str, Any], keys: tuple[str, ...]):
    for k in keys:
        if isinstance(record.get(k), (str, list)):
            return record[k]
    return None
