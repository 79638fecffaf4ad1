"""OpenAI chat-completion helpers shared by ``areno serve`` and the agentic rollout proxy:
message normalisation, chat-template tokenisation with ``tools``, the response envelope (with an
``areno`` metadata block carrying input tokens, response tokens and their log-probs) and
stop-string trimming.  Response shape follows ``areno/api/openai_chat.py:117-175`` of the reference.
"""

from __future__ import annotations

import json
import time
import uuid
from typing import Any

from .tokenizer import apply_chat_template_with_options, normalize_token_ids


def normalize_messages(messages: list[dict[str, Any]]) -> list[dict[str, Any]]:
    """``content: None`` becomes ``""``; stringified tool-call arguments become objects (templates
    iterate over them)."""
    out = []
    for m in messages:
        item = dict(m)
        if item.get("content") is None:
            item["content"] = ""
        calls = item.get("tool_calls")
        if isinstance(calls, list):
            fixed = []
            for c in calls:
                if isinstance(c, dict) and isinstance(c.get("function"), dict):
                    c = dict(c)
                    fn = dict(c["function"])
                    if isinstance(fn.get("arguments"), str):
                        try:
                            fn["arguments"] = json.loads(fn["arguments"] or "{}")
                        except json.JSONDecodeError:
                            pass
                    c["function"] = fn
                fixed.append(c)
            item["tool_calls"] = fixed
        out.append(item)
    return out


def messages_to_text(messages: list[dict[str, Any]]) -> str:
    return "\n".join(m["content"] for m in messages if isinstance(m.get("content"), str))


def first_user_text(messages: list[dict[str, Any]]) -> str:
    for m in messages:
        if m.get("role") == "user" and isinstance(m.get("content"), str):
            return m["content"]
    return messages_to_text(messages)


def _tools_for_template(tools: list[dict[str, Any]]) -> list[dict[str, Any]]:
    """Give every function a well-formed ``parameters`` object (some templates index into it)."""
    fixed = []
    for t in tools:
        if not isinstance(t, dict):
            continue
        t = dict(t)
        fn = t.get("function")
        if isinstance(fn, dict):
            fn = dict(fn)
            params = fn.get("parameters")
            if not isinstance(params, dict):
                fn["parameters"] = {"type": "object", "properties": {}}
            elif not isinstance(params.get("properties", {}), dict):
                fn["parameters"] = {**params, "properties": {}}
            t["function"] = fn
        fixed.append(t)
    return fixed


def messages_to_prompt_tokens(tokenizer: Any, messages: list[dict[str, Any]], *, tools: list[dict[str, Any]] | None = None,
                              fallback_prompt: str = "") -> list[int]:
    messages = normalize_messages(messages)
    if not getattr(tokenizer, "chat_template", None):
        return normalize_token_ids(tokenizer.encode(messages_to_text(messages) or fallback_prompt))
    base = {"tokenize": True, "add_generation_prompt": True}
    attempts = []
    if tools:
        attempts += [dict(base, tools=tools), dict(base, tools=_tools_for_template(tools))]
    attempts.append(base)
    # a template may reject ``tools`` in its own way (a TypeError for the keyword, a template error while it walks the
    # schema): every attempt but the last is allowed to fail, the plain rendering reports its own error
    for kwargs in attempts[:-1]:
        try:
            return normalize_token_ids(apply_chat_template_with_options(tokenizer, messages, **kwargs))
        except Exception:  # noqa: BLE001
            continue
    return normalize_token_ids(apply_chat_template_with_options(tokenizer, messages, **attempts[-1]))


def _decode(tokenizer: Any, ids: list[int], *, skip_special_tokens: bool) -> str:
    try:
        return tokenizer.decode(ids, skip_special_tokens=skip_special_tokens)
    except TypeError:
        return tokenizer.decode(ids)


def trim_stop_strings(text: str, stop: list[str]) -> tuple[str, bool]:
    cut = min((i for i in (text.find(s) for s in stop or []) if i >= 0), default=None)
    return (text, False) if cut is None else (text[:cut], True)


def build_chat_completion_response(*, tokenizer: Any, model: str, prompt_tokens: int, response_ids: list[list[int]],
                                   finish_reasons: list[str], tools: list[dict[str, Any]] | None = None,
                                   tool_choice: Any = None, tool_call_parser=None,
                                   parsed_tool_calls: list[list[dict[str, Any]]] | None = None,
                                   response_logprobs: list[list[float]] | None = None,
                                   include_areno_metadata: bool = False, input_tokens: list[int] | None = None,
                                   stop_strings: list[str] | None = None,
                                   include_logprobs: bool = False) -> dict[str, Any]:
    """``include_logprobs`` adds OpenAI's ``choices[i].logprobs.content``: one entry per generated token with the
    log-probability the sampler drew it at (no alternatives: ``top_logprobs`` stays empty)."""
    tools = list(tools or [])
    response_logprobs = response_logprobs or [[] for _ in response_ids]
    choices = []
    completion_tokens = 0
    for i, ids in enumerate(response_ids):
        raw = _decode(tokenizer, ids, skip_special_tokens=False)
        shown, stop_hit = trim_stop_strings(_decode(tokenizer, ids, skip_special_tokens=True), list(stop_strings or []))
        completion_tokens += len(ids)
        calls = parsed_tool_calls[i] if parsed_tool_calls is not None and i < len(parsed_tool_calls) else []
        if not calls and tools and tool_call_parser is not None:
            calls = tool_call_parser.parse(raw, tools, tool_choice).tool_calls
        finish = "stop" if stop_hit or finish_reasons[i] == "stop" else "length"
        message: dict[str, Any] = {"role": "assistant", "content": shown}
        if calls:
            message = {"role": "assistant", "content": None, "tool_calls": calls}
            finish = "tool_calls"
        choice: dict[str, Any] = {"index": i, "message": message, "finish_reason": finish}
        if include_logprobs:
            lps = response_logprobs[i] if i < len(response_logprobs) else []
            choice["logprobs"] = {"content": [
                {"token": _decode(tokenizer, [t], skip_special_tokens=False), "logprob": float(lp), "bytes": None,
                 "top_logprobs": []} for t, lp in zip(ids, lps)]}
        choices.append(choice)
    resp: dict[str, Any] = {
        "id": f"chatcmpl-{uuid.uuid4().hex}", "object": "chat.completion", "created": int(time.time()), "model": model,
        "choices": choices,
        "usage": {"prompt_tokens": prompt_tokens, "completion_tokens": completion_tokens,
                  "total_tokens": prompt_tokens + completion_tokens},
    }
    if include_areno_metadata:
        resp["areno"] = {"input_tokens": list(input_tokens or []),
                         "response_tokens": list(response_ids[0] if response_ids else []),
                         "response_logprobs": list(response_logprobs[0] if response_logprobs else [])}
    return resp
