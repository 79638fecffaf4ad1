"""Units of the agentic rollout path on the CPU, against a scripted trainer: batch expansion, trajectory metadata,
tool-call loss masks, merging of multi-turn and interleaved trajectories, prompt tokenisation through chat templates
(with tools, with templates that reject them), the proxy's request handling, reward records, the overlong-trajectory
filter of the policy trainer and loading of user agent files.  Behaviours follow the reference's
``tests/test_agentic_cpu.py``."""

from __future__ import annotations

import asyncio
import json
import logging
import threading
import urllib.error
import urllib.request
from types import SimpleNamespace

import pytest

from areno_b200.api import agentic
from areno_b200.api.agentic import (AgentBatch, AgentItem, AgentTrajectory, AgentTrajectoryTurn, LossMaskPolicy,
                                    RolloutSession, SampleAccumulator, common_prefix_len, load_agent_run_fn, maybe_await,
                                    render_messages, response_areno_metadata, response_tool_calls, tool_call_loss_mask,
                                    tool_results_from_messages)
from areno_b200.api.openai_chat import (build_chat_completion_response, first_user_text, messages_to_prompt_tokens,
                                        normalize_messages, trim_stop_strings)
from areno_b200.api.trainers.policy_only import PolicyOnlyTrainer


# ------------------------------------------------------------------------------------------------ test doubles

class WordTokenizer:
    """One token per whitespace-separated word; ids are handed out in order of first sight and decode exactly."""

    chat_template = None
    name_or_path = "words"
    eos_token_id = 0

    def __init__(self):
        self.vocab: dict[str, int] = {}
        self.words: list[str] = []

    def _id(self, word: str) -> int:
        if word not in self.vocab:
            self.vocab[word] = len(self.words) + 10
            self.words.append(word)
        return self.vocab[word]

    def encode(self, text, add_special_tokens=True):
        return [self._id(w) for w in str(text).split()]

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(self.words[int(t) - 10] for t in ids)


class ChatWordTokenizer(WordTokenizer):
    """Renders a conversation as ``<role> content`` per message; records what it was asked to render."""

    chat_template = "<role> content"

    def __init__(self):
        super().__init__()
        self.calls: list[dict] = []

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, **kw):
        self.calls.append({"messages": messages, "kw": kw, "tokenize": tokenize, "gen": add_generation_prompt})
        parts = []
        for m in messages:
            parts.append(f"<{m['role']}>")
            if not isinstance(m["content"], str):
                raise ValueError("content must be a string")
            parts.append(m["content"])
            for c in m.get("tool_calls") or []:
                parts.extend(f"{k}={v}" for k, v in c["function"]["arguments"].items())      # needs a mapping
        if add_generation_prompt:
            parts.append("<assistant>")
        text = " ".join(p for p in parts if p)
        return self.encode(text) if tokenize else text


class ScriptedTrainer:
    """The part of ``Trainer`` that a rollout session uses; completions come from a list of token rows."""

    def __init__(self, tokenizer=None, dp=1, script=None, delay_s=0.0):
        self.tokenizer = tokenizer or WordTokenizer()
        self._dp = dp
        self.script = list(script or [])
        self.delay_s = delay_s
        self.events: list[str] = []
        self.requests: list[tuple[list[int], int]] = []

    def get_tokenizer(self):
        return self.tokenizer

    def dp_size(self):
        return self._dp

    def begin_rollout_session(self):
        self.events.append("begin")

    def end_rollout_session(self):
        self.events.append("end")

    async def begin_rollout_session_async(self):
        self.events.append("begin_async")

    async def end_rollout_session_async(self):
        self.events.append("end_async")

    async def sync_rollout_session_async(self):
        self.events.append("sync")

    async def rollout_token_batch_async(self, prompt_tokens, n_samples, params):
        self.requests.append((list(prompt_tokens[0]), int(params.max_new_tokens)))
        if self.delay_s:
            await asyncio.sleep(self.delay_s)
        toks = self.script.pop(0) if self.script else self.tokenizer.encode("ok")
        toks = toks[:params.max_new_tokens]
        seq = SimpleNamespace(resp_tokens=list(toks), resp_logprobs=[-0.5] * len(toks))
        return [SimpleNamespace(sequences=[seq])]


class Params:
    def __init__(self, **kw):
        self.max_new_tokens, self.temperature, self.top_p = 8, 1.0, 1.0
        self.max_prompt_len = None
        self.__dict__.update(kw)

    def copy(self):
        return Params(**self.__dict__)


def _item(pi=0, si=0, prompt="p", record=None):
    return AgentItem(record=record if record is not None else {"answer": "a"}, prompt=prompt, input_tokens=[1],
                     prompt_index=pi, sample_index=si)


def _resp(tokens, logprobs=None, tool_calls=None, content="x"):
    msg = {"role": "assistant", "content": content}
    if tool_calls is not None:
        msg = {"role": "assistant", "content": None, "tool_calls": tool_calls}
    return {"choices": [{"message": msg}],
            "areno": {"response_tokens": list(tokens), "response_logprobs": list(logprobs or [-0.1] * len(tokens))}}


def _call(name, args, cid="c1"):
    return {"id": cid, "type": "function", "function": {"name": name, "arguments": args}}


# ------------------------------------------------------------------------------------------ batches and metadata

def test_agent_batch_expands_every_record_n_samples_times():
    batch = AgentBatch(records=[{"k": 1}, {"k": 2}], prompts=["a", "b"], input_tokens=[[1], [2, 3]], n_samples=3)
    items = list(batch.iter_samples())
    assert len(batch) == 6 and len(items) == 6
    assert [(i.prompt_index, i.sample_index) for i in items] == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), (1, 2)]
    assert items[4].prompt == "b" and items[4].input_tokens == [2, 3] and items[4].record == {"k": 2}


def test_agent_batch_from_prompt_batch_copies_records():
    src = SimpleNamespace(items=[SimpleNamespace(record={"q": 1}, prompt="p", input_tokens=(4, 5))])
    batch = AgentBatch.from_prompt_batch(src, n_samples=2)
    batch.records[0]["q"] = 9
    assert src.items[0].record == {"q": 1} and batch.input_tokens == [[4, 5]] and batch.n_samples == 2


def test_response_metadata_from_dicts_and_client_objects():
    meta = response_areno_metadata(_resp([1, 2]))
    assert meta["response_tokens"] == [1, 2]
    obj = SimpleNamespace(model_extra={"areno": {"response_tokens": [3], "response_logprobs": [-1.0]}})
    assert response_areno_metadata(obj)["response_tokens"] == [3]
    attr = SimpleNamespace(model_extra=None, areno={"response_tokens": [], "response_logprobs": []})
    assert response_areno_metadata(attr)["response_tokens"] == []


@pytest.mark.parametrize("bad,msg", [
    ({"choices": []}, "does not include"),
    ({"areno": {"response_tokens": [1]}}, "must include"),
    ({"areno": {"response_tokens": [1, 2], "response_logprobs": [0.0]}}, "length mismatch"),
])
def test_response_metadata_rejects_incomplete_blocks(bad, msg):
    with pytest.raises(ValueError, match=msg):
        response_areno_metadata(bad)


def test_turn_reads_tokens_logprobs_and_proxy_parsed_calls():
    turn = AgentTrajectoryTurn(item=_item(), messages=[{"role": "user", "content": "hi"}],
                               response=_resp([7, 8], [-0.25, -1], tool_calls=[_call("submit", {"b": 1, "a": 2})]))
    assert turn.response_tokens == [7, 8] and turn.response_logprobs == [-0.25, -1.0]
    assert turn.parsed_tool_calls == [{"id": "c1", "type": "function",
                                       "function": {"name": "submit", "arguments": '{"a": 2, "b": 1}'}}]
    # text that merely looks like a call is not parsed again by the agent side
    plain = AgentTrajectoryTurn(item=_item(), messages=[], response=_resp([1], content='{"tool": "submit"}'))
    assert plain.parsed_tool_calls == []


def test_response_tool_calls_skips_nameless_entries_and_fills_ids():
    resp = {"choices": [{"message": {"tool_calls": [{"function": {"arguments": "{}"}},
                                                    {"function": {"name": "go", "arguments": None}}]}}]}
    calls = response_tool_calls(resp)
    assert len(calls) == 1 and calls[0]["function"] == {"name": "go", "arguments": "{}"}
    assert calls[0]["id"].startswith("call_") and calls[0]["type"] == "function"
    assert response_tool_calls({"choices": []}) == [] and response_tool_calls({}) == []


def test_turn_without_response_keeps_explicit_fields():
    turn = AgentTrajectoryTurn(item=_item(), messages=[], response_tokens=[1, 2], response_logprobs=[-1.0, -2.0])
    assert turn.response is None and turn.response_tokens == [1, 2] and turn.parsed_tool_calls == []


# -------------------------------------------------------------------------------------------------- loss masks

def test_common_prefix_len():
    assert common_prefix_len([1, 2, 3], [1, 2, 4, 5]) == 2
    assert common_prefix_len([1, 2], [1, 2, 3]) == 2
    assert common_prefix_len([], [1]) == 0 and common_prefix_len([9], [1]) == 0


def test_tool_call_mask_is_all_true_without_a_sentinel():
    tok = WordTokenizer()
    ids = tok.encode('<tool_call> {"name": "f"} </tool_call>')
    assert tool_call_loss_mask(tok, ids) == [True] * len(ids)


@pytest.mark.parametrize("sentinel", ["<tool_response>", "<|tool_response>"])
def test_tool_call_mask_stops_at_an_echoed_tool_response(sentinel):
    tok = WordTokenizer()
    ids = tok.encode(f"<tool_call> call </tool_call> {sentinel} invented result")
    mask = tool_call_loss_mask(tok, ids)
    assert mask == [True, True, True, False, False, False]


def test_tool_call_mask_decodes_once_and_survives_broken_tokenizers():
    class Counting(WordTokenizer):
        decodes = 0

        def decode(self, ids, skip_special_tokens=True):
            Counting.decodes += 1
            return super().decode(ids)

    tok = Counting()
    ids = tok.encode("a b <tool_response> c")
    assert tool_call_loss_mask(tok, ids) == [True, True, False, False] and Counting.decodes == 1

    class Broken:
        def decode(self, ids):
            raise RuntimeError("no decoder")

    assert tool_call_loss_mask(Broken(), [1, 2, 3]) == [True, True, True]


def test_policy_masks_tool_calls_and_text_independently():
    tok = WordTokenizer()
    call_turn = AgentTrajectoryTurn(item=_item(0, 0), messages=[{"role": "user", "content": "q"}],
                                    response=_resp(tok.encode("call it"), tool_calls=[_call("f", "{}")]))
    text_turn = AgentTrajectoryTurn(item=_item(1, 0), messages=[{"role": "user", "content": "q"}],
                                    response=_resp(tok.encode("plain words")))
    on = SampleAccumulator(tok, LossMaskPolicy())
    assert on.add_turn(call_turn).response_loss_mask == [True, True]
    assert on.add_turn(text_turn).response_loss_mask == [True, True]
    off_calls = SampleAccumulator(tok, LossMaskPolicy(assistant_tool_calls=False))
    assert off_calls.add_turn(call_turn).response_loss_mask == [False, False]
    assert off_calls.add_turn(text_turn).response_loss_mask == [True, True]
    off_text = SampleAccumulator(tok, LossMaskPolicy(assistant_text=False))
    assert off_text.add_turn(call_turn).response_loss_mask == [True, True]
    s = off_text.add_turn(text_turn)
    assert s.response_loss_mask == [False, False] and s.response_mask_row[-2:] == [True, True]
    assert s.loss_mask_row[-2:] == [False, False]


# ------------------------------------------------------------------------------------------- merging of turns

def _two_turns(tok, item, first_words, tool_words, second_words):
    msgs = [{"role": "user", "content": item.prompt}]
    t1 = AgentTrajectoryTurn(item=item, messages=list(msgs), response=_resp(tok.encode(first_words)))
    msgs = msgs + [{"role": "assistant", "content": first_words}, {"role": "tool", "name": "t", "content": tool_words}]
    t2 = AgentTrajectoryTurn(item=item, messages=list(msgs), response=_resp(tok.encode(second_words)))
    return t1, t2


def test_multi_turn_calls_merge_into_one_row():
    tok = WordTokenizer()
    item = _item(prompt="what now")
    t1, t2 = _two_turns(tok, item, "first answer", "tool output", "second answer here")
    acc = SampleAccumulator(tok, LossMaskPolicy())
    acc.add_turn(t1)
    s = acc.add_turn(t2)
    assert len(acc.samples) == 1
    # without a chat template the prompt is the concatenated message text: the second prompt starts with the first row
    assert tok.decode(s.token_row) == "what now first answer tool output second answer here"
    assert s.response_mask_row == [False, False, True, True, False, False, True, True, True]
    assert s.loss_mask_row == s.response_mask_row
    assert s.rollout_logprobs_row == [0.0, 0.0, -0.1, -0.1, 0.0, 0.0, -0.1, -0.1, -0.1]
    assert s.response_text == "first answer\nsecond answer here" and s.last_response_text == "second answer here"
    assert len(s.response_tokens) == 5 and len(s.response_logprobs) == 5 and len(s.response_loss_mask) == 5
    assert [e.type for e in s.trace] == ["request", "assistant_text", "finish"] * 2
    assert s.messages[-1]["role"] == "tool"


def test_interleaved_trajectories_stay_with_their_items():
    tok = WordTokenizer()
    a, b = _item(0, 0, "alpha prompt"), _item(0, 1, "alpha prompt")
    c = _item(1, 0, "beta prompt")
    a1, a2 = _two_turns(tok, a, "a one", "ra", "a two")
    b1, b2 = _two_turns(tok, b, "b one", "rb", "b two")
    c1, _ = _two_turns(tok, c, "c only", "rc", "unused")
    acc = SampleAccumulator(tok, LossMaskPolicy())
    for turn in (a1, b1, c1, b2, a2):
        acc.add_turn(turn)
    assert [(s.item.prompt_index, s.item.sample_index) for s in acc.samples] == [(0, 0), (0, 1), (1, 0)]
    sa, sb, sc = acc.samples
    assert tok.decode(sa.token_row) == "alpha prompt a one ra a two"
    assert tok.decode(sb.token_row) == "alpha prompt b one rb b two"
    assert tok.decode(sc.token_row) == "beta prompt c only"
    assert sa.last_response_text == "a two" and sb.last_response_text == "b two"


def test_session_accumulate_accepts_trajectories_turn_lists_and_singletons():
    tok = WordTokenizer()
    session = RolloutSession(ScriptedTrainer(tok), sampling_params=Params())
    t1, t2 = _two_turns(tok, _item(0, 0, "q"), "x", "r", "y")
    u1, _ = _two_turns(tok, _item(1, 0, "q"), "z", "r", "w")
    assert len(session.accumulate(AgentTrajectory(turns=[t1, t2]))) == 1
    assert len(session.accumulate([AgentTrajectory(turns=[t1, t2]), [u1]])) == 2


def test_normalize_trajectories_shapes():
    t = AgentTrajectoryTurn(item=_item(), messages=[], response=_resp([1]))
    norm = PolicyOnlyTrainer._normalize_trajectories
    assert norm(t) == [[t]]
    traj = AgentTrajectory(turns=[t])
    assert norm(traj) == [traj]
    assert norm([t, traj, [t, t]]) == [[t], traj, [t, t]]


# ------------------------------------------------------------------------------------- messages and templates

def test_normalize_messages_makes_templates_safe_and_leaves_the_input_alone():
    src = [{"role": "assistant", "content": None,
            "tool_calls": [_call("inspect", '{"path": ".", "depth": 3}'), _call("raw", "not json"), "odd"]}]
    out = normalize_messages(src)
    assert out[0]["content"] == ""
    assert out[0]["tool_calls"][0]["function"]["arguments"] == {"path": ".", "depth": 3}
    assert out[0]["tool_calls"][1]["function"]["arguments"] == "not json" and out[0]["tool_calls"][2] == "odd"
    assert src[0]["content"] is None and isinstance(src[0]["tool_calls"][0]["function"]["arguments"], str)


def test_prompt_tokens_pass_tools_to_the_template():
    tok = ChatWordTokenizer()
    tools = [{"type": "function", "function": {"name": "choose"}}]
    ids = messages_to_prompt_tokens(tok, [{"role": "user", "content": "pick one"}], tools=tools)
    assert tok.decode(ids) == "<user> pick one <assistant>"
    assert tok.calls[0]["kw"] == {"tools": tools} and len(tok.calls) == 1


def test_prompt_tokens_render_tool_history_with_null_content_and_string_arguments():
    tok = ChatWordTokenizer()
    msgs = [{"role": "user", "content": "go"},
            {"role": "assistant", "content": None, "tool_calls": [_call("f", '{"x": 1}')]},
            {"role": "tool", "tool_call_id": "c1", "content": "done"}]
    ids = messages_to_prompt_tokens(tok, msgs)
    assert tok.decode(ids) == "<user> go <assistant> x=1 <tool> done <assistant>"


@pytest.mark.parametrize("exc", [TypeError("unexpected keyword 'tools'"), ValueError("template: tools unsupported")])
def test_prompt_tokens_fall_back_when_the_template_rejects_tools(exc):
    class Rejecting(ChatWordTokenizer):
        def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, **kw):
            if "tools" in kw:
                self.calls.append({"rejected": kw})
                raise exc
            return super().apply_chat_template(messages, tokenize, add_generation_prompt, **kw)

    tok = Rejecting()
    ids = messages_to_prompt_tokens(tok, [{"role": "user", "content": "hi"}], tools=[{"type": "function", "function": {"name": "f"}}])
    assert tok.decode(ids) == "<user> hi <assistant>"
    assert [("rejected" in c) for c in tok.calls] == [True, True, False]     # as given, with filled schemas, without


def test_prompt_tokens_report_the_plain_template_error():
    class Failing(ChatWordTokenizer):
        def apply_chat_template(self, *a, **kw):
            raise ValueError("broken template")

    with pytest.raises(ValueError, match="broken template"):
        messages_to_prompt_tokens(Failing(), [{"role": "user", "content": "hi"}], tools=[{"type": "function"}])


def test_prompt_tokens_without_a_template_use_text_or_the_fallback():
    tok = WordTokenizer()
    assert tok.decode(messages_to_prompt_tokens(tok, [{"role": "user", "content": "a b"}])) == "a b"
    assert tok.decode(messages_to_prompt_tokens(tok, [{"role": "user", "content": None}], fallback_prompt="fb")) == "fb"


def test_render_messages_uses_the_template_then_plain_text():
    tok = ChatWordTokenizer()
    msgs = [{"role": "user", "content": "q"}, {"role": "assistant", "content": None, "tool_calls": [_call("f", '{"k": 2}')]}]
    assert render_messages(tok, msgs) == "<user> q <assistant> k=2"
    assert tok.calls[-1]["tokenize"] is False and tok.calls[-1]["gen"] is False

    class Failing(ChatWordTokenizer):
        def apply_chat_template(self, *a, **kw):
            raise ValueError("nope")

    assert render_messages(Failing(), [{"role": "user", "content": "q"}, {"role": "assistant", "content": "r"}]) == "q\nr"
    assert render_messages(WordTokenizer(), [{"role": "user", "content": "only"}]) == "only"


def test_first_user_text_and_stop_strings():
    assert first_user_text([{"role": "system", "content": "s"}, {"role": "user", "content": "u"}]) == "u"
    assert first_user_text([{"role": "system", "content": "s"}]) == "s"
    assert trim_stop_strings("abc END def STOP", ["STOP", "END"]) == ("abc ", True)
    assert trim_stop_strings("abc", ["X"]) == ("abc", False) and trim_stop_strings("abc", []) == ("abc", False)


def test_chat_completion_envelope_carries_the_trajectory_block():
    tok = WordTokenizer()
    ids = tok.encode("final words")
    resp = build_chat_completion_response(tokenizer=tok, model="m", prompt_tokens=3, response_ids=[ids],
                                          finish_reasons=["length"], response_logprobs=[[-1.0, -2.0]],
                                          include_areno_metadata=True, input_tokens=[5, 6, 7])
    assert resp["choices"][0]["message"] == {"role": "assistant", "content": "final words"}
    assert resp["choices"][0]["finish_reason"] == "length"
    assert resp["usage"] == {"prompt_tokens": 3, "completion_tokens": 2, "total_tokens": 5}
    assert resp["areno"] == {"input_tokens": [5, 6, 7], "response_tokens": ids, "response_logprobs": [-1.0, -2.0]}
    calls = [_call("f", "{}")]
    with_calls = build_chat_completion_response(tokenizer=tok, model="m", prompt_tokens=1, response_ids=[ids],
                                                finish_reasons=["stop"], parsed_tool_calls=[calls])
    assert with_calls["choices"][0]["finish_reason"] == "tool_calls" and "areno" not in with_calls
    assert with_calls["choices"][0]["message"] == {"role": "assistant", "content": None, "tool_calls": calls}
    stopped = build_chat_completion_response(tokenizer=tok, model="m", prompt_tokens=1, response_ids=[ids],
                                             finish_reasons=["length"], stop_strings=["words"])
    assert stopped["choices"][0] == {"index": 0, "message": {"role": "assistant", "content": "final "},
                                     "finish_reason": "stop"}


# ------------------------------------------------------------------------------------------------ the session

def test_session_parallelism_defaults_to_the_data_parallel_size():
    assert RolloutSession(ScriptedTrainer(dp=8), sampling_params=Params()).max_running_prompts == 8
    assert RolloutSession(ScriptedTrainer(dp=8), sampling_params=Params(), max_running_prompts=3).max_running_prompts == 3
    assert RolloutSession(ScriptedTrainer(dp=2), sampling_params=Params(), max_running_prompts=0).max_running_prompts == 1

    class NoDp(ScriptedTrainer):
        def dp_size(self):
            raise RuntimeError("not initialised")

    assert RolloutSession(NoDp(), sampling_params=Params()).max_running_prompts == 1


def test_session_contexts_own_the_backend_lifecycle():
    trainer = ScriptedTrainer()
    with RolloutSession(trainer, sampling_params=Params()) as s:
        with pytest.raises(RuntimeError):
            RolloutSession(trainer, sampling_params=Params(), proxy=False).base_url
        assert trainer.events == ["begin"] and s.max_running_prompts == 1
    assert trainer.events == ["begin", "end"]

    async def run():
        async with RolloutSession(trainer, sampling_params=Params(), proxy=False) as s:
            await s.sync_rollout_session_async()
            s.finish_requests()
            assert s._server is None
    asyncio.run(run())
    assert trainer.events[2:] == ["begin_async", "sync", "end_async"]


def test_session_ends_the_backend_session_when_the_body_raises():
    trainer = ScriptedTrainer()

    async def run():
        async with RolloutSession(trainer, sampling_params=Params()):
            raise KeyError("agent failed")

    with pytest.raises(KeyError):
        asyncio.run(run())
    assert trainer.events == ["begin_async", "end_async"]


def test_proxy_server_bounds_its_handler_threads():
    assert agentic._ProxyServer.request_queue_size >= 1024 and agentic._ProxyServer.daemon_threads
    server = agentic._ProxyServer(("127.0.0.1", 0), agentic.BaseHTTPRequestHandler, max_threads=3)
    try:
        assert server._slots._initial_value == 3
    finally:
        server.server_close()


def _post(url, body, raw=None):
    data = raw if raw is not None else json.dumps(body).encode()
    req = urllib.request.Request(url, data=data, headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=30) as resp:
            return resp.status, json.loads(resp.read())
    except urllib.error.HTTPError as exc:
        return exc.code, json.loads(exc.read() or b"{}")


def test_proxy_http_status_codes_and_request_overrides():
    tok = WordTokenizer()
    trainer = ScriptedTrainer(tok, script=[tok.encode("one two three four")])

    async def run():
        loop = asyncio.get_running_loop()
        async with RolloutSession(trainer, sampling_params=Params(max_new_tokens=8), timeout_s=30) as s:
            url = s.get_base_url()
            assert url.startswith("http://127.0.0.1:") and url.endswith("/v1")
            call = lambda *a, **k: loop.run_in_executor(None, lambda: _post(*a, **k))       # noqa: E731
            assert (await call(url + "/models", {}))[0] == 404
            assert (await call(url + "/chat/completions", None, raw=b"{not json"))[0] == 400
            status, err = await call(url + "/chat/completions", {"messages": [{"role": "user", "content": "x"}], "stream": True})
            assert status == 400 and "streaming" in err["error"]["message"]
            assert (await call(url + "/chat/completions", {"messages": []}))[0] == 400
            status, ok = await call(url + "/chat/completions",
                                    {"messages": [{"role": "user", "content": "count for me"}], "max_tokens": 3,
                                     "temperature": 0.5, "top_p": 0.9, "model": "named"})
            assert status == 200 and ok["model"] == "named"
            assert tok.decode(ok["areno"]["response_tokens"]) == "one two three"
            assert ok["areno"]["response_logprobs"] == [-0.5] * 3
            assert tok.decode(ok["areno"]["input_tokens"]) == "count for me"
            assert ok["choices"][0]["message"]["content"] == "one two three"
            assert ok["usage"] == {"prompt_tokens": 3, "completion_tokens": 3, "total_tokens": 6}
    asyncio.run(run())
    assert trainer.requests == [(tok.encode("count for me"), 3)]


def test_proxy_answers_an_overlong_prompt_without_a_rollout():
    tok = WordTokenizer()
    trainer = ScriptedTrainer(tok)
    session = RolloutSession(trainer, sampling_params=Params(max_prompt_len=2), proxy=False)
    resp = asyncio.run(session.complete_chat({"messages": [{"role": "user", "content": "far too many words"}]}))
    assert trainer.requests == []
    assert resp["choices"][0]["finish_reason"] == "length" and resp["choices"][0]["message"]["content"] == ""
    assert resp["usage"]["prompt_tokens"] == 4 and resp["usage"]["max_sequence_len"] == 2
    assert resp["areno"] == {"input_tokens": [], "response_tokens": [], "response_logprobs": []}
    # a turn built from it is empty but well formed
    turn = AgentTrajectoryTurn(item=_item(), messages=[{"role": "user", "content": "far too many words"}], response=resp)
    assert turn.response_tokens == []


def test_proxy_returns_parsed_tool_calls_for_declared_tools():
    tok = WordTokenizer()
    text = '{"tool": "lookup", "arguments": {"q": "cats"}}'
    trainer = ScriptedTrainer(tok, script=[tok.encode(text)])
    session = RolloutSession(trainer, sampling_params=Params(max_new_tokens=32), proxy=False)
    tools = [{"type": "function", "function": {"name": "lookup", "parameters": {"type": "object", "properties": {"q": {"type": "string"}}}}}]
    resp = asyncio.run(session.complete_chat({"messages": [{"role": "user", "content": "find cats"}], "tools": tools}))
    choice = resp["choices"][0]
    assert choice["finish_reason"] == "tool_calls" and choice["message"]["content"] is None
    fn = choice["message"]["tool_calls"][0]["function"]
    assert fn["name"] == "lookup" and json.loads(fn["arguments"]) == {"q": "cats"}
    # agent side: the turn takes the proxy's parse, the reward record shows call and (later) the tool's answer
    item = _item(record={"answer": "cats"}, prompt="find cats")
    turn = AgentTrajectoryTurn(item=item, messages=[{"role": "user", "content": "find cats"}], response=resp, tools=tools)
    sample = session.accumulate([[turn]])[0]
    rec = session.reward_record(sample)
    assert rec.tool_calls == [{"name": "lookup", "arguments": fn["arguments"]}]
    assert rec.messages[-1]["tool_calls"][0]["function"]["name"] == "lookup" and rec.answer == "cats"
    assert [e.type for e in rec.trace] == ["request", "assistant_tool_call", "finish"]


def test_proxy_times_out_a_stuck_rollout():
    trainer = ScriptedTrainer(delay_s=5.0)
    session = RolloutSession(trainer, sampling_params=Params(), proxy=False, timeout_s=0.05)
    with pytest.raises(TimeoutError, match="timed out"):
        asyncio.run(session.complete_chat({"messages": [{"role": "user", "content": "x"}]}))


def test_a_client_that_gives_up_does_not_cancel_other_requests():
    tok = WordTokenizer()
    trainer = ScriptedTrainer(tok, delay_s=0.3)

    async def run():
        loop = asyncio.get_running_loop()
        async with RolloutSession(trainer, sampling_params=Params(), timeout_s=30) as s:
            url = s.get_base_url() + "/chat/completions"
            body = {"messages": [{"role": "user", "content": "x"}]}

            def impatient():
                req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
                try:
                    urllib.request.urlopen(req, timeout=0.05)
                except Exception:        # noqa: BLE001  (socket timeout: the client walks away)
                    return "gave up"
                return "answered"

            quitter = loop.run_in_executor(None, impatient)
            patient = loop.run_in_executor(None, _post, url, body)
            assert await quitter == "gave up"
            status, resp = await patient
            assert status == 200 and resp["areno"]["response_tokens"]
            await asyncio.sleep(0.4)          # the abandoned request still runs to its end on the loop
    asyncio.run(run())
    assert len(trainer.requests) == 2


# --------------------------------------------------------------------------------------------- reward records

def test_reward_record_lists_tool_results_before_the_first_finish():
    tok = ChatWordTokenizer()
    session = RolloutSession(ScriptedTrainer(tok), sampling_params=Params(), proxy=False)
    item = _item(record={"solutions": ["s"], "id": 3}, prompt="ask")
    msgs = [{"role": "user", "content": "ask"}]
    t1 = AgentTrajectoryTurn(item=item, messages=list(msgs), response=_resp(tok.encode("calling"), tool_calls=[_call("f", '{"a": 1}')]))
    msgs += [{"role": "assistant", "content": None, "tool_calls": [_call("f", '{"a": 1}')]},
             {"role": "tool", "name": "f", "tool_call_id": "c1", "content": "result text"}]
    t2 = AgentTrajectoryTurn(item=item, messages=list(msgs), response=_resp(tok.encode("the end")))
    sample = session.accumulate([AgentTrajectory(turns=[t1, t2])])[0]
    rec = session.reward_record(sample)
    assert rec.answer == ["s"] and rec.source_record == {"solutions": ["s"], "id": 3}
    assert rec.final_answer == "the end" and rec.completion == "calling\nthe end"
    assert rec.tool_results == [{"name": "f", "tool_call_id": "c1", "content": "result text"}]
    assert rec.tool_calls == [{"name": "f", "arguments": '{"a": 1}'}]
    types = [e.type for e in rec.trace]
    assert types.index("tool_result") < types.index("finish") and types.count("tool_result") == 1
    assert rec.trace[types.index("tool_result")].metadata == {"tool_call_id": "c1"}
    assert rec.messages[-1] == {"role": "assistant", "content": "the end"}
    assert rec.rendered_completion.endswith("<assistant> the end") and "<tool> result text" in rec.rendered_completion
    assert rec.metadata == {"prompt_index": 0, "sample_index": 0}
    assert rec.tokens == sample.response_tokens and rec.loss_mask == sample.response_loss_mask
    assert tool_results_from_messages([{"role": "user", "content": "x"}]) == []


def test_train_batch_without_a_reward_function_has_no_rewards():
    tok = WordTokenizer()
    session = RolloutSession(ScriptedTrainer(tok), sampling_params=Params(), proxy=False)
    t1, _ = _two_turns(tok, _item(record={"answer": "z"}, prompt="q"), "r s", "x", "y")
    samples = session.accumulate([[t1]])
    batch = session.build_train_batch(samples, None)
    assert batch.rewards is None and batch.records == [{"answer": "z"}]
    assert batch.token_rows == [tok.encode("q r s")] and batch.response_masks == [[False, True, True]]
    scored = session.build_train_batch(samples, lambda rec: len(rec.tokens))
    assert scored.rewards == [2.0]
    scored.token_rows[0].append(99)                     # the batch owns its rows
    assert samples[0].token_row == tok.encode("q r s")


# --------------------------------------------------------------------------- overlong trajectories (policy trainer)

def _policy(limit_cfg=None, model_len=None):
    p = object.__new__(PolicyOnlyTrainer)
    p.logger = logging.getLogger("test.agentic.filter")
    p.config = SimpleNamespace(max_context_len=limit_cfg)
    if model_len is None:
        p.areno = SimpleNamespace()
    else:
        p.areno = SimpleNamespace(model_context_len=lambda: model_len)
    return p


def _sample_of(tok, pi, n_prompt, n_resp):
    words = " ".join(f"p{pi}_{i}" for i in range(n_prompt))
    turn = AgentTrajectoryTurn(item=_item(pi, 0, words), messages=[{"role": "user", "content": words}],
                               response=_resp(tok.encode(" ".join(f"r{pi}_{i}" for i in range(n_resp)))))
    return SampleAccumulator(tok, LossMaskPolicy()).add_turn(turn)


def test_overlong_trajectories_are_dropped_with_a_warning(caplog):
    tok = WordTokenizer()
    short, long_ = _sample_of(tok, 0, 1, 1), _sample_of(tok, 1, 4, 3)
    with caplog.at_level(logging.WARNING):
        kept, dropped, diag = _policy(model_len=4)._filter_overlong([short, long_], Params(max_prompt_len=2, max_new_tokens=2))
    assert kept == [short] and dropped == 1
    assert diag["max_context_len"] == 4 and diag["filtered"] == 1 and diag["kept"] == 1 and diag["total"] == 2
    assert diag["top"][0]["tokens"] == 7 and diag["top"][0]["prompt_idx"] == 1 and diag["top"][0]["response_tokens"] == 3
    assert "agentic trajectory filtered" in caplog.text and "max_context_len=4" in caplog.text


def test_the_filter_measures_the_whole_row_not_the_prompt_limit():
    tok = WordTokenizer()
    s = _sample_of(tok, 0, 7, 3)
    kept, dropped, diag = _policy(model_len=10)._filter_overlong([s], Params(max_prompt_len=2, max_new_tokens=5))
    assert kept == [s] and dropped == 0 and diag["max_context_len"] == 10 and diag["top"] == []


def test_the_configured_context_length_wins_when_it_is_smaller():
    tok = WordTokenizer()
    s = _sample_of(tok, 0, 4, 2)
    kept, dropped, diag = _policy(limit_cfg=5, model_len=100)._filter_overlong([s], Params())
    assert kept == [] and dropped == 1 and diag["max_context_len"] == 5 and diag["top"][0]["tokens"] == 6
    assert _policy(limit_cfg=50, model_len=8)._context_limit(Params()) == 8


def test_no_limit_means_no_filter():
    tok = WordTokenizer()
    s = _sample_of(tok, 0, 40, 20)
    assert _policy()._filter_overlong([s], Params()) == ([s], 0, {})


def test_the_filter_counts_merged_turns():
    tok = WordTokenizer()
    t1, t2 = _two_turns(tok, _item(prompt="a b"), "c", "d", "e f")
    acc = SampleAccumulator(tok, LossMaskPolicy())
    acc.add_turn(t1)
    merged = acc.add_turn(t2)
    assert len(merged.token_row) == 6
    kept, dropped, diag = _policy(limit_cfg=5)._filter_overlong([merged], Params())
    assert kept == [] and dropped == 1
    assert diag["top"][0]["tokens"] == 6 and diag["top"][0]["tool_results"] == 1 and diag["top"][0]["assistant_messages"] == 1


def test_filter_diagnostics_text():
    diag = {"max_context_len": 8, "total": 2, "kept": 0, "filtered": 2, "min_tokens": 12, "p50_tokens": 12,
            "p90_tokens": 20, "max_tokens": 20,
            "top": [{"prompt_idx": 1, "sample_idx": 0, "tokens": 20, "messages": 6, "assistant_messages": 3,
                     "tool_results": 2, "response_tokens": 5, "trace_events": 4, "prompt": "build kit"}]}
    text = PolicyOnlyTrainer._format_filter_diagnostics(diag)
    for part in ("max_context_len=8", "tokens[min/p50/p90/max]=12/12/20/20", "prompt_idx=1", "tool_results=2", "prompt='build kit'"):
        assert part in text
    assert "no context-length diagnostics" in PolicyOnlyTrainer._format_filter_diagnostics({})


# -------------------------------------------------------------------------------------------- user agent files

def test_load_agent_run_fn(tmp_path):
    good = tmp_path / "agent.py"
    good.write_text("async def run_agent(session, batch):\n    return [session, batch]\n")
    fn = load_agent_run_fn(str(good))
    assert asyncio.run(maybe_await(fn(1, 2))) == [1, 2]
    bad = tmp_path / "no_fn.py"
    bad.write_text("run_agent = 3\n")
    with pytest.raises(ValueError, match="run_agent"):
        load_agent_run_fn(str(bad))


def test_maybe_await_passes_plain_values_through():
    async def run():
        fut = asyncio.get_running_loop().create_future()
        fut.set_result(5)
        return await maybe_await(4), await maybe_await(fut)
    assert asyncio.run(run()) == (4, 5)


def test_threads_of_the_proxy_share_one_event_loop():
    """Concurrent HTTP requests are all served by coroutines of the loop that opened the session."""
    tok = WordTokenizer()
    trainer = ScriptedTrainer(tok, delay_s=0.05)
    seen = set()
    orig = trainer.rollout_token_batch_async

    async def spy(*a, **k):
        seen.add(threading.get_ident())
        return await orig(*a, **k)

    trainer.rollout_token_batch_async = spy

    async def run():
        loop = asyncio.get_running_loop()
        async with RolloutSession(trainer, sampling_params=Params(), timeout_s=30) as s:
            url = s.get_base_url() + "/chat/completions"
            jobs = [loop.run_in_executor(None, _post, url, {"messages": [{"role": "user", "content": f"q{i}"}]}) for i in range(6)]
            out = await asyncio.gather(*jobs)
            assert [st for st, _ in out] == [200] * 6
        return threading.get_ident()
    main = asyncio.run(run())
    assert seen == {main} and len(trainer.requests) == 6
