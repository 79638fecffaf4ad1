"""Unit tests of the SDK's pure-Python pieces: tool-call parsers, agentic row accumulation and loss masks, chat
helpers, tokenizer helpers, GAE, data utilities.  No model, no GPU."""

from __future__ import annotations

import json
from types import SimpleNamespace

import pytest

from .helpers import FakeTokenizer

TOOLS = [{"type": "function", "function": {"name": "place", "parameters": {
    "type": "object", "properties": {"cell": {"type": "integer"}}, "required": ["cell"]}}},
    {"type": "function", "function": {"name": "pick", "parameters": {
        "type": "object", "properties": {"colour": {"type": "string", "enum": ["Red", "Green"]}}, "required": ["colour"]}}}]


def _args(call):
    return json.loads(call["function"]["arguments"])


# ----------------------------------------------------------------------------------------- tool-call parsers
def test_json_parser_accepts_objects_lists_and_code_fences_and_ignores_unknown_tools():
    from areno_b200.api.tool_call_parser import get_tool_call_parser

    p = get_tool_call_parser("json")
    r = p.parse('{"name": "place", "arguments": {"cell": 4}}', TOOLS, None)
    assert r.normal_text == "" and r.tool_calls[0]["function"]["name"] == "place" and _args(r.tool_calls[0]) == {"cell": 4}
    r = p.parse('```json\n[{"name": "place", "arguments": {"cell": 1}}, {"name": "pick", "arguments": {"colour": "Red"}}]\n```',
                TOOLS, None)
    assert [c["function"]["name"] for c in r.tool_calls] == ["place", "pick"]
    r = p.parse('{"name": "rm_rf", "arguments": {}}', TOOLS, None)
    assert r.tool_calls == [] and "rm_rf" in r.normal_text                   # not an offered tool: plain text
    assert p.parse("just words", [], None).normal_text == "just words"       # no tools offered: nothing is parsed


def test_forced_tool_with_single_enum_argument_is_recovered_from_plain_text():
    from areno_b200.api.tool_call_parser import get_tool_call_parser

    forced = {"type": "function", "function": {"name": "pick"}}
    r = get_tool_call_parser("json").parse("I would answer green here.", TOOLS, forced)
    assert len(r.tool_calls) == 1 and _args(r.tool_calls[0]) == {"colour": "Green"}    # canonical spelling of the enum
    r = get_tool_call_parser("json").parse("colour = red, final", TOOLS, forced)
    assert _args(r.tool_calls[0]) == {"colour": "Red"}
    r = get_tool_call_parser("json").parse("green is nice but I will not say which", TOOLS, forced)
    assert r.tool_calls == []                                        # only explicit choices are recovered


def test_qwen_parser_reads_json_and_function_eq_blocks_and_keeps_leading_text():
    from areno_b200.api.tool_call_parser import get_tool_call_parser

    p = get_tool_call_parser("qwen")
    text = 'Let me move.\n<tool_call>\n{"name": "place", "arguments": {"cell": 7}}\n</tool_call>'
    r = p.parse(text, TOOLS, None)
    assert r.normal_text == "Let me move." and _args(r.tool_calls[0]) == {"cell": 7}
    text = "<tool_call><function=place><parameter=cell>3</parameter></function></tool_call>"
    r = p.parse(text, TOOLS, None)
    assert _args(r.tool_calls[0]) == {"cell": 3}                               # scalars are typed
    two = text + "\n" + text.replace("3", "5")
    assert [_args(c)["cell"] for c in p.parse(two, TOOLS, None).tool_calls] == [3, 5]


def test_minicpm_and_gemma_parsers():
    from areno_b200.api.tool_call_parser import get_tool_call_parser

    m = get_tool_call_parser("minicpm")
    r = m.parse('thinking <function name="place"><param name="cell">2</param></function>', TOOLS, None)
    assert r.normal_text == "thinking" and _args(r.tool_calls[0]) == {"cell": 2}
    g = get_tool_call_parser("gemma4")
    r = g.parse('ok <|tool_call>call:pick{colour:<|"|>Red<|"|>}<tool_call|>', TOOLS, None)
    assert r.normal_text == "ok" and _args(r.tool_calls[0]) == {"colour": "Red"}
    r = g.parse("<|tool_call>call:place{cell:8}<tool_call|><|tool_call>call:unknown{a:1}<tool_call|>", TOOLS, None)
    assert len(r.tool_calls) == 1 and _args(r.tool_calls[0]) == {"cell": 8}


def test_parser_is_inferred_from_template_path_and_config(tmp_path):
    from areno_b200.api.tool_call_parser import infer_tool_call_parser_name

    def trainer(template="", path=""):
        tok = SimpleNamespace(chat_template=template, name_or_path=path)
        return SimpleNamespace(get_tokenizer=lambda: tok, _model_path=path)

    assert infer_tool_call_parser_name(trainer("... <tool_call> ...")) == "qwen"
    assert infer_tool_call_parser_name(trainer("... <|tool_call> ...")) == "gemma4"
    assert infer_tool_call_parser_name(trainer(path="/models/MiniCPM-V-4_6")) == "minicpm"
    assert infer_tool_call_parser_name(trainer()) == "json"
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"model_type": "gemma4", "architectures": ["Gemma4ForConditionalGeneration"]}))
    assert infer_tool_call_parser_name(trainer(path=str(d))) == "gemma4"


def test_custom_parser_can_be_registered():
    from areno_b200.api.tool_call_parser import (ToolCallParseResult, get_tool_call_parser, list_tool_call_parsers,
                                                 make_tool_call, register_tool_call_parser)

    class Shout:
        name = "shout"

        def parse(self, content, tools, tool_choice):
            return ToolCallParseResult("", [make_tool_call("place", {"cell": len(content)})])

    register_tool_call_parser("shout", Shout)
    assert "shout" in list_tool_call_parsers()
    assert _args(get_tool_call_parser("shout").parse("abc", TOOLS, None).tool_calls[0]) == {"cell": 3}
    assert get_tool_call_parser("no-such-parser").name == "json"       # unknown names fall back to the JSON parser


# ----------------------------------------------------------------------------------------- agentic accumulation
def _item(pi=0, si=0, prompt="what now"):
    from areno_b200.api.agentic import AgentItem

    return AgentItem(record={"prompt": prompt}, prompt=prompt, input_tokens=[4, 5], prompt_index=pi, sample_index=si)


def _response(tokens, text=None, calls=None):
    msg = {"role": "assistant", "content": text, "tool_calls": calls or []}
    return {"choices": [{"message": msg}],
            "areno": {"response_tokens": list(tokens), "response_logprobs": [-0.5] * len(tokens)}}


def test_response_metadata_is_validated():
    from areno_b200.api.agentic import AgentTrajectoryTurn, response_areno_metadata, response_tool_calls

    with pytest.raises(ValueError):
        response_areno_metadata({"choices": []})
    with pytest.raises(ValueError):
        response_areno_metadata({"areno": {"response_tokens": [1, 2], "response_logprobs": [0.0]}})
    obj = SimpleNamespace(model_extra={"areno": {"response_tokens": [1], "response_logprobs": [-1.0]}})
    assert response_areno_metadata(obj)["response_tokens"] == [1]              # OpenAI client objects work too
    calls = response_tool_calls(_response([1], calls=[{"function": {"name": "place", "arguments": {"cell": 1}}},
                                                       {"function": {"arguments": "{}"}}]))
    assert len(calls) == 1 and calls[0]["function"]["arguments"] == '{"cell": 1}' and calls[0]["id"].startswith("call_")
    turn = AgentTrajectoryTurn(item=_item(), messages=[{"role": "user", "content": "hi"}], response=_response([7, 8, 9]))
    assert turn.response_tokens == [7, 8, 9] and turn.response_logprobs == [-0.5] * 3


def test_turns_of_one_sample_merge_into_one_row_with_masks():
    from areno_b200.api.agentic import AgentTrajectoryTurn, LossMaskPolicy, SampleAccumulator

    tok = FakeTokenizer()
    acc = SampleAccumulator(tok, LossMaskPolicy())
    first = [{"role": "user", "content": "play a move"}]
    call = [{"id": "c1", "type": "function", "function": {"name": "place", "arguments": '{"cell": 4}'}}]
    t1 = AgentTrajectoryTurn(item=_item(), messages=first, response=_response(tok.encode("i place four"), calls=call), tools=TOOLS)
    s = acc.add_turn(t1)
    n_prompt = len(s.token_row) - 3
    assert s.response_mask_row == [False] * n_prompt + [True] * 3 and s.loss_mask_row[n_prompt:] == [True] * 3
    second = first + [{"role": "assistant", "content": None, "tool_calls": call},
                      {"role": "tool", "tool_call_id": "c1", "name": "place", "content": '{"result": "continue"}'}]
    t2 = AgentTrajectoryTurn(item=_item(), messages=second, response=_response(tok.encode("done now"), text="done now"))
    merged = acc.add_turn(t2)
    assert merged is s and len(acc.samples) == 1
    assert merged.response_tokens == tok.encode("i place four") + tok.encode("done now")
    assert len(merged.token_row) == len(merged.response_mask_row) == len(merged.loss_mask_row) == len(merged.rollout_logprobs_row)
    assert sum(merged.response_mask_row) == 5                       # only generated tokens count as response
    assert merged.last_response_text == "done now" and merged.last_tool_calls == []
    # a different sample index starts a new row
    other = acc.add_turn(AgentTrajectoryTurn(item=_item(si=1), messages=first, response=_response([9], text="x")))
    assert other is not s and len(acc.samples) == 2


def test_loss_mask_policy_and_tool_response_echo_cut():
    from areno_b200.api.agentic import AgentTrajectoryTurn, LossMaskPolicy, SampleAccumulator, tool_call_loss_mask

    tok = FakeTokenizer()
    call = [{"id": "c1", "type": "function", "function": {"name": "place", "arguments": "{}"}}]
    msgs = [{"role": "user", "content": "go"}]
    acc = SampleAccumulator(tok, LossMaskPolicy(assistant_tool_calls=False))
    s = acc.add_turn(AgentTrajectoryTurn(item=_item(), messages=msgs, response=_response(tok.encode("a b"), calls=call)))
    assert not any(s.loss_mask_row)                                # tool-call spans switched off
    acc = SampleAccumulator(tok, LossMaskPolicy(assistant_text=False))
    s = acc.add_turn(AgentTrajectoryTurn(item=_item(), messages=msgs, response=_response(tok.encode("a b"), text="a b")))
    assert not any(s.loss_mask_row)
    ids = tok.encode("call it <tool_response> invented result")
    mask = tool_call_loss_mask(tok, ids)
    assert mask == [True, True] + [False] * (len(ids) - 2)         # nothing after an echoed tool-response marker is trained on


def test_common_prefix_and_tool_results():
    from areno_b200.api.agentic import common_prefix_len, tool_results_from_messages

    assert common_prefix_len([1, 2, 3], [1, 2, 4, 5]) == 2 and common_prefix_len([], [1]) == 0 and common_prefix_len([1], [1]) == 1
    msgs = [{"role": "user", "content": "u"}, {"role": "tool", "name": "t", "tool_call_id": "c", "content": "r"}]
    assert tool_results_from_messages(msgs) == [{"name": "t", "tool_call_id": "c", "content": "r"}]


def test_agent_batch_expands_prompts_into_samples():
    from areno_b200.api.agentic import AgentBatch

    batch = AgentBatch(records=[{"a": 1}, {"a": 2}], prompts=["p0", "p1"], input_tokens=[[1], [2, 3]], n_samples=3)
    items = list(batch.iter_samples())
    assert len(batch) == 6 and [(i.prompt_index, i.sample_index) for i in items] == [(p, s) for p in range(2) for s in range(3)]
    assert items[4].prompt == "p1" and items[4].record == {"a": 2}


# ----------------------------------------------------------------------------------------- chat / tokenizer helpers
def test_chat_helpers():
    from areno_b200.api.openai_chat import first_user_text, messages_to_text, normalize_messages, trim_stop_strings

    call = {"id": "c", "type": "function", "function": {"name": "place", "arguments": '{"cell": 2}'}}
    msgs = normalize_messages([{"role": "system", "content": "s"}, {"role": "user", "content": "hello there"},
                               {"role": "assistant", "content": None, "tool_calls": [call]}])
    assert msgs[2]["content"] == "" and msgs[2]["tool_calls"][0]["function"]["arguments"] == {"cell": 2}
    assert call["function"]["arguments"] == '{"cell": 2}'                  # the caller's objects are not modified
    assert first_user_text(msgs) == "hello there"
    assert messages_to_text(msgs).splitlines()[:2] == ["s", "hello there"]
    assert trim_stop_strings("abc STOP def", ["STOP"]) == ("abc ", True)
    assert trim_stop_strings("abc", ["STOP"]) == ("abc", False)


def test_token_id_normalisation_and_generation_prompt():
    from areno_b200.api.tokenizer import encode_generation_prompt, looks_chat_formatted, normalize_token_ids

    assert normalize_token_ids([1, 2, 3]) == [1, 2, 3]
    assert normalize_token_ids([[4, 5]]) == [4, 5]                          # a batch of one
    with pytest.raises(TypeError):
        normalize_token_ids([[1], [2]])                                      # a real batch is refused
    assert normalize_token_ids(SimpleNamespace(input_ids=[6])) == [6]
    assert looks_chat_formatted("<|im_start|>user\nhi<|im_end|>") and not looks_chat_formatted("plain question")
    tok = FakeTokenizer()
    assert encode_generation_prompt(tok, "what is two plus two") == tok.encode("what is two plus two")


def test_gae_matches_the_recurrence():
    from areno_b200.api.advantages import compute_gae

    rewards, values, gamma, lam = [0.0, 0.0, 1.0], [0.2, 0.4, 0.6], 0.9, 0.8
    adv, ret = compute_gae(rewards, values, gamma=gamma, lam=lam)
    want, nxt_adv, nxt_v = [], 0.0, 0.0
    for r, v in zip(reversed(rewards), reversed(values)):
        delta = r + gamma * nxt_v - v
        nxt_adv = delta + gamma * lam * nxt_adv
        want.append(nxt_adv)
        nxt_v = v
    want.reverse()
    assert list(adv) == pytest.approx(want) and list(ret) == pytest.approx([a + v for a, v in zip(want, values)])


def test_data_utils_build_prompt_response_rows():
    from areno_b200.api.data_utils import first_text, has_any, prompt_response_to_tokens_and_mask

    tok = FakeTokenizer()
    tokens, mask = prompt_response_to_tokens_and_mask("what is it", "it is this", tok, eos_token_id=2)
    n_prompt = len(tok.encode("what is it"))
    assert tokens[:n_prompt] == tok.encode("what is it") and tokens[-1] == 2
    assert mask[:n_prompt] == [True] * n_prompt and not any(mask[n_prompt:])       # True marks prompt positions
    assert has_any({"question": "q"}, ("prompt", "question")) and not has_any({"x": 1}, ("prompt",))
    assert first_text({"question": " q "}, ("prompt", "question")).strip() == "q"


# ----------------------------------------------------------------------------------------- rewards
def test_reward_functions_are_loaded_from_files_and_records_carry_the_row(tmp_path):
    from areno_b200.api.rewards import compute_group_advantages, load_reward_fn, make_reward_record

    good = tmp_path / "r.py"
    good.write_text("def reward_fn(record):\n    return float(record.completion.strip() == str(record.answer))\n")
    fn = load_reward_fn(str(good))
    rec = make_reward_record(prompt="2+2", completion=" 4 ", source_record={"answer": 4, "extra": "kept"}, answer=4,
                             tokens=[7], logprobs=[-0.25], loss_mask=[True], metadata={"turns": 1})
    assert fn(rec) == 1.0 and rec.final_answer == " 4 " and rec.source_record["extra"] == "kept"
    assert rec.tokens == [7] and rec.logprobs == [-0.25] and rec.metadata == {"turns": 1} and rec.tool_calls == []
    bad = tmp_path / "bad.py"
    bad.write_text("reward_fn = 3\n")
    with pytest.raises(ValueError, match="reward_fn"):
        load_reward_fn(str(bad))
    adv = compute_group_advantages([1.0, 0.0, 0.0, 1.0])
    assert adv == pytest.approx([1.0, -1.0, -1.0, 1.0], abs=1e-4) and sum(adv) == pytest.approx(0.0, abs=1e-6)
    assert compute_group_advantages([0.5, 0.5, 0.5]) == pytest.approx([0.0, 0.0, 0.0])      # no signal: no gradient
