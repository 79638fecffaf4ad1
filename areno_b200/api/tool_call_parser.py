"""Tool-call parsers for the OpenAI-compatible endpoints.

A parser turns model-native tool-call text into OpenAI ``message.tool_calls`` entries plus the
leftover assistant text.  Parsers are registered by name (``json``, ``qwen``, ``gemma4``,
``minicpm``); ``infer_tool_call_parser_name`` picks one from the chat template / model path /
``config.json``.  Formats covered (as in ``areno/api/tool_call_parser.py:20-527`` of the reference):

* ``json``    - a JSON object / list / ``{"tool_calls": [...]}`` anywhere in the text; with a single
  (or forced) tool whose only enum argument can be read from free text, that value is used;
* ``qwen``    - ``<tool_call> {json} </tool_call>`` blocks, or ``<function=name><parameter=k>v</parameter>``
  inside them;
* ``gemma4``  - ``<|tool_call>call:name{key:value,...}<tool_call|>`` with ``<|"|>`` string quotes;
* ``minicpm`` - ``<function name="..."><param name="...">v</param></function>`` (plus the qwen block form).
"""

from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Protocol


@dataclass
class ToolCallParseResult:
    normal_text: str
    tool_calls: list[dict[str, Any]] = field(default_factory=list)


class ToolCallParser(Protocol):
    name: str

    def parse(self, content: str, tools: list[dict[str, Any]], tool_choice: Any) -> ToolCallParseResult:
        ...


_PARSERS: dict[str, type] = {}


def register_tool_call_parser(name: str, parser_cls: type) -> None:
    _PARSERS[name.lower()] = parser_cls


def get_tool_call_parser(name: str | None) -> ToolCallParser:
    return _PARSERS.get((name or "json").lower(), JsonToolCallParser)()


def list_tool_call_parsers() -> list[str]:
    return sorted(_PARSERS)


# ------------------------------------------------------------------ tool schema helpers
def tool_function(tool: Any) -> dict[str, Any] | None:
    """OpenAI function schema from chat (``{"type": "function", "function": {...}}``) or flat syntax."""
    if not isinstance(tool, dict):
        return None
    if isinstance(tool.get("function"), dict):
        return tool["function"]
    if isinstance(tool.get("name"), str):
        return {"name": tool["name"], "description": tool.get("description"), "parameters": tool.get("parameters")}
    return None


class _Schema:
    """The tools offered on a request and the caller's ``tool_choice``."""

    def __init__(self, tools: list[dict[str, Any]], tool_choice: Any):
        self.functions = [f for f in (tool_function(t) for t in tools or []) if f and isinstance(f.get("name"), str)]
        self.names = {f["name"] for f in self.functions}
        forced = None
        if isinstance(tool_choice, dict):
            fn = tool_choice.get("function")
            if isinstance(fn, dict) and isinstance(fn.get("name"), str):
                forced = fn["name"]
        if forced is None and len(tools or []) == 1 and self.functions:
            forced = self.functions[0]["name"]
        self.forced = forced

    def allows(self, name: str) -> bool:
        return name == self.forced if self.forced is not None else name in self.names

    def single_enum_argument(self, name: str):
        for f in self.functions:
            if f["name"] != name:
                continue
            props = (f.get("parameters") or {}).get("properties") if isinstance(f.get("parameters"), dict) else None
            if not isinstance(props, dict):
                return None
            enums = [(k, s["enum"]) for k, s in props.items()
                     if isinstance(s, dict) and isinstance(s.get("enum"), list) and s["enum"]]
            return enums[0] if len(enums) == 1 else None
        return None


def make_tool_call(name: str, arguments: dict[str, Any]) -> dict[str, Any]:
    return {"id": f"call_{uuid.uuid4().hex[:24]}", "type": "function",
            "function": {"name": name, "arguments": json.dumps(arguments, ensure_ascii=False, separators=(",", ":"))}}


# ------------------------------------------------------------------------- JSON family
def _loads_lenient(text: str):
    text = text.strip()
    try:
        return json.loads(text)
    except json.JSONDecodeError:
        pass
    for opener, closer in (("{", "}"), ("[", "]")):
        a, b = text.find(opener), text.rfind(closer)
        if a != -1 and b > a:
            try:
                return json.loads(text[a:b + 1])
            except json.JSONDecodeError:
                continue
    return None


def _call_from_object(obj: Any, default_name: str | None):
    if not isinstance(obj, dict):
        return None
    fn = obj.get("function")
    if isinstance(fn, dict):
        name = fn.get("name") or obj.get("name") or default_name
        args = fn.get("arguments", obj.get("arguments", {}))
    else:
        name = obj.get("name") or default_name
        args = obj["arguments"] if "arguments" in obj else obj
    if not isinstance(name, str) or not name:
        return None
    if isinstance(args, str):
        args = _loads_lenient(args)
    if not isinstance(args, dict):
        return None
    return name, dict(args)


def _json_calls(text: str, schema: _Schema) -> list[dict[str, Any]]:
    obj = _loads_lenient(text)
    if obj is None:
        return []
    if isinstance(obj, dict) and isinstance(obj.get("tool_calls"), list):
        raws = obj["tool_calls"]
    elif isinstance(obj, list):
        raws = obj
    else:
        raws = [obj]
    calls = []
    for raw in raws:
        parsed = _call_from_object(raw, schema.forced)
        if parsed and schema.allows(parsed[0]):
            calls.append(make_tool_call(*parsed))
    return calls


def _enum_value_from_text(text: str, key: str, values: list[Any]):
    by_lower = {str(v).lower(): v for v in values}
    if not by_lower:
        return None
    alts = "|".join(re.escape(v) for v in by_lower)
    k = re.escape(key)
    patterns = (
        rf'["\']?{k}["\']?\s*[:=]\s*["\']?\b({alts})\b',
        rf"<(?:{k}|move|action)>\s*({alts})\s*</(?:{k}|move|action)>",
        rf"\b(?:choose|select|play|move|slide|go|answer|direction)\s*(?:is|:|=|to)?\s*\b({alts})\b",
    )
    for pat in patterns:
        found = re.findall(pat, text, flags=re.IGNORECASE)
        if found:
            return by_lower[str(found[-1]).lower()]
    return None


class JsonToolCallParser:
    name = "json"

    def parse(self, content, tools, tool_choice) -> ToolCallParseResult:
        if not tools:
            return ToolCallParseResult(normal_text=content)
        schema = _Schema(tools, tool_choice)
        calls = _json_calls(content, schema)
        if calls:
            return ToolCallParseResult("", calls)
        if schema.forced is not None:
            enum = schema.single_enum_argument(schema.forced)
            if enum is not None:
                value = _enum_value_from_text(content, *enum)
                if value is not None:
                    return ToolCallParseResult("", [make_tool_call(schema.forced, {enum[0]: value})])
        return ToolCallParseResult(normal_text=content)


# --------------------------------------------------------------------- angle-bracket forms
_BLOCK_RE = re.compile(r"<tool_call>\s*(.*?)\s*</tool_call>", re.DOTALL | re.IGNORECASE)
_FUNC_EQ_RE = re.compile(r"<function=([^>\s]+)>\s*(.*?)</function>", re.DOTALL | re.IGNORECASE)
_PARAM_EQ_RE = re.compile(r"<parameter=([^>\s]+)>\s*(.*?)</parameter>", re.DOTALL | re.IGNORECASE)


def _scalar(text: str):
    text = re.sub(r"<\|[^>]+?\|>", "", text).strip()
    low = text.lower()
    if low in ("true", "false"):
        return low == "true"
    for cast in (int, float):
        try:
            return cast(text)
        except ValueError:
            pass
    return text


def _function_eq_calls(text: str, schema: _Schema) -> list[dict[str, Any]]:
    calls = []
    for name, body in _FUNC_EQ_RE.findall(text):
        if schema.allows(name):
            calls.append(make_tool_call(name.strip(), {k.strip(): _scalar(v) for k, v in _PARAM_EQ_RE.findall(body)}))
    return calls


class QwenToolCallParser(JsonToolCallParser):
    name = "qwen"

    def parse(self, content, tools, tool_choice) -> ToolCallParseResult:
        schema = _Schema(tools, tool_choice)
        calls: list[dict[str, Any]] = []
        for block in _BLOCK_RE.findall(content):
            calls += _json_calls(block, schema)
            calls += _function_eq_calls(block, schema)
        if calls:
            return ToolCallParseResult(content[: content.lower().find("<tool_call>")].strip(), calls)
        return super().parse(content, tools, tool_choice)


class MiniCPMToolCallParser(JsonToolCallParser):
    name = "minicpm"
    _func = re.compile(r"<function\s+name=[\"']([^\"']+)[\"']\s*>(.*?)</function>", re.DOTALL | re.IGNORECASE)
    _param = re.compile(r"<param\s+name=[\"']([^\"']+)[\"']\s*>(.*?)</param>", re.DOTALL | re.IGNORECASE)

    def parse(self, content, tools, tool_choice) -> ToolCallParseResult:
        schema = _Schema(tools, tool_choice)
        calls: list[dict[str, Any]] = []
        for block in _BLOCK_RE.findall(content):
            calls += _function_eq_calls(block, schema)
        for name, body in self._func.findall(content):
            if schema.allows(name):
                calls.append(make_tool_call(name.strip(), {k.strip(): _scalar(v) for k, v in self._param.findall(body)}))
        if calls:
            starts = [i for i in (content.find("<tool_call>"), content.find("<function")) if i >= 0]
            return ToolCallParseResult(content[: min(starts)].strip() if starts else "", calls)
        return super().parse(content, tools, tool_choice)


# ------------------------------------------------------------------------------ gemma4
_GQ = '<|"|>'


class _GemmaValueReader:
    """Recursive-descent reader of Gemma's ``key:value`` argument syntax (quotes are ``<|"|>``)."""

    def __init__(self, text: str):
        self.s = text
        self.i = 0

    def _ws(self):
        while self.i < len(self.s) and self.s[self.i].isspace():
            self.i += 1

    def _quoted(self) -> str:
        self.i += len(_GQ)
        end = self.s.find(_GQ, self.i)
        if end == -1:
            end = len(self.s)
        out = self.s[self.i:end]
        self.i = min(len(self.s), end + len(_GQ))
        return out

    def _bare(self, stops: str) -> str:
        start = self.i
        while self.i < len(self.s) and self.s[self.i] not in stops:
            self.i += 1
        return self.s[start:self.i].strip()

    def key(self) -> str:
        self._ws()
        if self.s.startswith(_GQ, self.i):
            k = self._quoted()
        else:
            k = self._bare(":,}").strip("\"'")
        self._ws()
        return k

    def value(self):
        self._ws()
        if self.s.startswith(_GQ, self.i):
            return self._quoted()
        if self.i < len(self.s) and self.s[self.i] == "{":
            self.i += 1
            return self.members("}")
        if self.i < len(self.s) and self.s[self.i] == "[":
            self.i += 1
            items = []
            while True:
                self._ws()
                if self.i >= len(self.s):
                    break
                if self.s[self.i] == "]":
                    self.i += 1
                    break
                items.append(self.value())
                self._ws()
                if self.i < len(self.s) and self.s[self.i] == ",":
                    self.i += 1
            return items
        raw = self._bare(",}]")
        if raw in ("true", "false"):
            return raw == "true"
        if raw == "null":
            return None
        for cast in (int, float):
            try:
                return cast(raw)
            except ValueError:
                pass
        return raw

    def members(self, closer: str | None) -> dict[str, Any]:
        out: dict[str, Any] = {}
        while True:
            self._ws()
            if self.i >= len(self.s):
                break
            if closer and self.s[self.i] == closer:
                self.i += 1
                break
            k = self.key()
            if self.i < len(self.s) and self.s[self.i] == ":":
                self.i += 1
                v = self.value()
                if k:
                    out[k] = v
            self._ws()
            if self.i < len(self.s) and self.s[self.i] == ",":
                self.i += 1
            elif self.i < len(self.s) and closer and self.s[self.i] == closer:
                self.i += 1
                break
            elif self.i < len(self.s) and self.s[self.i] not in ",}":
                self.i += 1  # skip a stray character rather than loop forever
        return out


def _gemma_call(inner: str):
    if not inner.startswith("call:"):
        return None
    brace = inner.find("{")
    if brace == -1:
        return None
    name = inner[len("call:"):brace].strip()
    reader = _GemmaValueReader(inner[brace + 1:])
    return name, reader.members("}")


class Gemma4ToolCallParser(JsonToolCallParser):
    name = "gemma4"
    _start, _end = "<|tool_call>", "<tool_call|>"

    def parse(self, content, tools, tool_choice) -> ToolCallParseResult:
        schema = _Schema(tools, tool_choice)
        calls = []
        pos = 0
        while True:
            a = content.find(self._start, pos)
            if a == -1:
                break
            b = content.find(self._end, a)
            if b == -1:
                break
            parsed = _gemma_call(content[a + len(self._start):b].strip())
            if parsed and schema.allows(parsed[0]):
                calls.append(make_tool_call(*parsed))
            pos = b + len(self._end)
        if calls:
            return ToolCallParseResult(content[: content.find(self._start)].strip(), calls)
        return super().parse(content, tools, tool_choice)


# -------------------------------------------------------------------------- inference
def _model_type_words(model_path: str) -> str:
    if not model_path:
        return ""
    cfg = Path(model_path) / "config.json"
    if not cfg.exists():
        return ""
    try:
        data = json.loads(cfg.read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError):
        return ""
    parts = [str(data.get("model_type", "")), str((data.get("text_config") or {}).get("model_type", "")),
             " ".join(str(a) for a in data.get("architectures") or [])]
    return " ".join(p.lower() for p in parts if p)


def infer_tool_call_parser_name(trainer: Any) -> str:
    """Pick a parser from the tokenizer's chat template, the model path and ``config.json``."""
    try:
        tokenizer = trainer.get_tokenizer()
    except Exception:
        tokenizer = None
    template = str(getattr(tokenizer, "chat_template", "") or "").lower()
    model_path = str(getattr(trainer, "_model_path", "") or getattr(getattr(trainer, "_ctx", None), "model_path", "")
                     or getattr(tokenizer, "name_or_path", "") or "").lower()
    hay = " ".join([template, model_path, _model_type_words(model_path)])
    if "<|tool_call>" in template or "gemma4" in hay or "gemma-4" in hay:
        return "gemma4"
    if "minicpm" in hay:
        return "minicpm"
    if "<tool_call>" in template or "qwen" in hay:
        return "qwen"
    return "json"


for _cls in (JsonToolCallParser, QwenToolCallParser, Gemma4ToolCallParser, MiniCPMToolCallParser):
    register_tool_call_parser(_cls.name, _cls)
