"""Tool-call parsers: each supported model syntax to OpenAI ``tool_calls`` entries, the tool-choice rules that
filter them, value typing, leftovers, malformed input, and parser selection."""

from __future__ import annotations

import json

import pytest

from areno_b200.api.tool_call_parser import (ToolCallParseResult, get_tool_call_parser, infer_tool_call_parser_name,
                                             list_tool_call_parsers, make_tool_call, tool_function)

WEATHER = {"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}}}}
MOVE = {"type": "function", "function": {"name": "move", "parameters": {
    "type": "object", "properties": {"direction": {"type": "string", "enum": ["up", "down", "left", "right"]}}}}}
FLAT = {"name": "lookup", "description": "flat syntax", "parameters": {"type": "object", "properties": {}}}


def _args(call):
    return json.loads(call["function"]["arguments"])


def _names(result):
    return [c["function"]["name"] for c in result.tool_calls]


def test_registry_lists_the_four_syntaxes_and_defaults_to_json():
    assert {"json", "qwen", "gemma4", "minicpm"} <= set(list_tool_call_parsers())
    assert get_tool_call_parser(None).name == "json" and get_tool_call_parser("QWEN").name == "qwen"
    assert get_tool_call_parser("no-such-parser").name == "json"


def test_tool_function_accepts_chat_and_flat_schemas():
    assert tool_function(WEATHER)["name"] == "get_weather" and tool_function(FLAT)["name"] == "lookup"
    assert tool_function("not a dict") is None and tool_function({"type": "function"}) is None


def test_make_tool_call_serialises_compact_json_with_a_fresh_id():
    a, b = make_tool_call("f", {"x": 1, "s": "é"}), make_tool_call("f", {"x": 1, "s": "é"})
    assert a["type"] == "function" and a["function"] == {"name": "f", "arguments": '{"x":1,"s":"é"}'}
    assert a["id"].startswith("call_") and a["id"] != b["id"]


@pytest.mark.parametrize("text", [
    '{"name": "get_weather", "arguments": {"city": "Oslo", "days": 2}}',
    'Sure. {"name": "get_weather", "arguments": "{\\"city\\": \\"Oslo\\", \\"days\\": 2}"} Done.',
    '[{"function": {"name": "get_weather", "arguments": {"city": "Oslo", "days": 2}}}]',
    '{"tool_calls": [{"name": "get_weather", "arguments": {"city": "Oslo", "days": 2}}]}'])
def test_json_parser_reads_objects_lists_and_wrapped_calls(text):
    r = get_tool_call_parser("json").parse(text, [WEATHER, MOVE], "auto")
    assert _names(r) == ["get_weather"] and _args(r.tool_calls[0]) == {"city": "Oslo", "days": 2} and r.normal_text == ""


def test_json_parser_drops_calls_to_tools_that_were_not_offered_or_not_forced():
    p = get_tool_call_parser("json")
    text = '[{"name": "get_weather", "arguments": {"city": "a"}}, {"name": "rm_rf", "arguments": {}}]'
    assert _names(p.parse(text, [WEATHER, MOVE], "auto")) == ["get_weather"]
    forced = {"type": "function", "function": {"name": "move"}}
    assert p.parse(text, [WEATHER, MOVE], forced).tool_calls == []            # only the forced tool may be called
    assert p.parse(text, [], "auto") == ToolCallParseResult(normal_text=text)  # no tools offered: plain text


def test_a_bare_argument_object_calls_the_single_offered_tool():
    r = get_tool_call_parser("json").parse('{"city": "Lima"}', [WEATHER], "auto")
    assert _names(r) == ["get_weather"] and _args(r.tool_calls[0]) == {"city": "Lima"}


@pytest.mark.parametrize("text,expect", [("direction: LEFT", "left"), ("<move>down</move>", "down"),
                                         ("I will go right now", "right"), ("first up ... finally I choose down", "down")])
def test_single_enum_argument_is_read_from_free_text(text, expect):
    r = get_tool_call_parser("json").parse(text, [MOVE], "auto")
    assert _names(r) == ["move"] and _args(r.tool_calls[0]) == {"direction": expect}


def test_free_text_without_a_recognisable_value_stays_text():
    r = get_tool_call_parser("json").parse("sideways maybe", [MOVE], "auto")
    assert r.tool_calls == [] and r.normal_text == "sideways maybe"
    # two offered tools and no forced choice: free text is never turned into a call
    assert get_tool_call_parser("json").parse("go left", [MOVE, WEATHER], "auto").tool_calls == []


def test_qwen_blocks_json_and_function_parameter_forms_with_leading_text():
    text = ('Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Rome"}}\n</tool_call>\n'
            "<tool_call><function=move><parameter=direction>up</parameter></function></tool_call>")
    r = get_tool_call_parser("qwen").parse(text, [WEATHER, MOVE], "auto")
    assert _names(r) == ["get_weather", "move"] and r.normal_text == "Let me check."
    assert _args(r.tool_calls[1]) == {"direction": "up"}


def test_qwen_parameter_values_are_typed():
    text = ("<tool_call><function=get_weather><parameter=city>Paris</parameter><parameter=days>3</parameter>"
            "<parameter=metric>true</parameter><parameter=scale>1.5</parameter></function></tool_call>")
    r = get_tool_call_parser("qwen").parse(text, [WEATHER], "auto")
    assert _args(r.tool_calls[0]) == {"city": "Paris", "days": 3, "metric": True, "scale": 1.5}


def test_qwen_falls_back_to_plain_json_and_ignores_unclosed_blocks():
    p = get_tool_call_parser("qwen")
    assert _names(p.parse('{"name": "move", "arguments": {"direction": "up"}}', [MOVE], "auto")) == ["move"]
    r = p.parse("<tool_call>{\"name\": \"get_weather\"", [WEATHER, MOVE], "auto")
    assert r.tool_calls == [] and r.normal_text.startswith("<tool_call>")


def test_minicpm_function_tags_and_qwen_style_blocks():
    p = get_tool_call_parser("minicpm")
    text = 'ok <function name="get_weather"><param name="city">Kyoto</param><param name="days">4</param></function>'
    r = p.parse(text, [WEATHER], "auto")
    assert _names(r) == ["get_weather"] and _args(r.tool_calls[0]) == {"city": "Kyoto", "days": 4} and r.normal_text == "ok"
    r = p.parse("<tool_call><function=move><parameter=direction>left</parameter></function></tool_call>", [MOVE], "auto")
    assert _args(r.tool_calls[0]) == {"direction": "left"}
    assert p.parse('<function name="unknown"></function>', [WEATHER, MOVE], "auto").tool_calls == []


def test_gemma4_call_syntax_with_nested_values_and_quotes():
    q = '<|"|>'
    text = (f"thinking... <|tool_call>call:get_weather{{city:{q}New York{q},days:2,opts:{{units:{q}c{q},hourly:false}},"
            f"tags:[{q}a{q},3,null]}}<tool_call|> trailing")
    r = get_tool_call_parser("gemma4").parse(text, [WEATHER], "auto")
    assert _names(r) == ["get_weather"] and r.normal_text == "thinking..."
    assert _args(r.tool_calls[0]) == {"city": "New York", "days": 2, "opts": {"units": "c", "hourly": False},
                                     "tags": ["a", 3, None]}


def test_gemma4_several_calls_and_garbage_between_markers():
    p = get_tool_call_parser("gemma4")
    text = "<|tool_call>call:move{direction:up}<tool_call|><|tool_call>not a call<tool_call|><|tool_call>call:move{direction:down}<tool_call|>"
    r = p.parse(text, [MOVE], "auto")
    assert [_args(c)["direction"] for c in r.tool_calls] == ["up", "down"]
    # no closing marker: not a gemma call; with several tools on offer the free-text fallback does not apply either
    assert p.parse("<|tool_call>call:move{direction:up}", [MOVE, WEATHER], "auto").tool_calls == []


def test_parser_is_inferred_from_template_path_or_config(tmp_path):
    class Tok:
        def __init__(self, template="", path=""):
            self.chat_template, self.name_or_path = template, path

    class Trainer:
        def __init__(self, tok=None, path=""):
            self._tok, self._model_path = tok, path

        def get_tokenizer(self):
            if self._tok is None:
                raise RuntimeError("not initialised")
            return self._tok

    assert infer_tool_call_parser_name(Trainer(Tok("... <tool_call> ..."))) == "qwen"
    assert infer_tool_call_parser_name(Trainer(Tok("... <|tool_call> ..."))) == "gemma4"
    assert infer_tool_call_parser_name(Trainer(Tok(path="/models/Qwen3-8B"))) == "qwen"
    assert infer_tool_call_parser_name(Trainer(None, "/models/MiniCPM-V-4_6")) == "minicpm"
    assert infer_tool_call_parser_name(Trainer(None)) == "json"
    d = tmp_path / "ckpt"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"model_type": "x", "text_config": {"model_type": "gemma4_text"}}))
    assert infer_tool_call_parser_name(Trainer(Tok(), str(d))) == "gemma4"
    (d / "config.json").write_text("{broken json")
    assert infer_tool_call_parser_name(Trainer(Tok(), str(d))) == "json"
