"""Units of ``areno serve`` on the CPU: how the command builds its engine, request defaults, chat templates that take
tools and the thinking switch, stop ids from the tokenizer's vocabulary, prompts that do not fit, failures of the
engine, and shutdown.  Behaviours follow the reference's ``tests/test_serve_cli_cpu.py``."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
from click.testing import CliRunner
from fastapi.testclient import TestClient

from areno_b200.cli import serve
from areno_b200.engine.config import RuntimeConfig
from tests.helpers import FakeTokenizer
from tests.test_serve_cpu import ScriptedEngine


class TemplateTokenizer(FakeTokenizer):
    chat_template = "[role] content"

    def __init__(self):
        super().__init__()
        self.calls = []

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, **kw):
        self.calls.append({"messages": messages, **kw})
        text = " ".join(f"[{m['role']}] {m['content']}" for m in messages) + " [assistant]"
        return self.encode(text)


def test_the_command_builds_the_engine_from_its_options(monkeypatch):
    seen = {}

    def fake_from_pretrained(model, **kw):
        seen.update(model=model, **kw)
        return ScriptedEngine([5])

    monkeypatch.setattr("areno_b200.engine.api.ArenoEngine.from_pretrained", staticmethod(fake_from_pretrained))
    tok = FakeTokenizer()
    app = serve.create_app(model_path="some/model", tp_size=2, world_size=4, max_running_prompts=9, eager_decode=True,
                           attn_backend="native", kv_dtype="fp8", tokenizer=tok, chat_template_enable_thinking=False)
    assert seen["model"] == "some/model" and (seen["tp_size"], seen["dp_size"], seen["devices"]) == (2, 2, [0, 1, 2, 3])
    rt = seen["runtime_config"]
    assert isinstance(rt, RuntimeConfig) and rt.eager_decode and rt.attn_backend == "native" and rt.kv_dtype == "fp8"
    assert seen["max_running_seqs"] == 9 and seen["loss_fn"] is serve.serve_loss_fn
    with pytest.raises(RuntimeError, match="does not support training"):
        seen["loss_fn"]({}, None)
    state = app.state.areno_serve
    assert state.max_model_len == 256 and state.max_running_prompts == 9
    assert getattr(tok, "_areno_chat_template_enable_thinking") is False
    for bad in (dict(world_size=0), dict(tp_size=0), dict(world_size=3, tp_size=2)):
        with pytest.raises(ValueError):
            serve.create_app(model_path="m", tokenizer=tok, engine=object(), **bad)


def test_command_line_defaults_and_checks(monkeypatch):
    opts = {p.name: p.default for p in serve.serve_command.params}
    assert (opts["max_running_prompts"], opts["default_max_tokens"], opts["tp_size"], opts["world_size"]) == (16, 1024, 1, 1)
    assert (opts["port"], opts["attn_backend"], opts["kv_dtype"]) == (8000, "flash", "bf16")
    runner = CliRunner()
    assert "--max-running-prompts must be positive" in runner.invoke(
        serve.serve_command, ["--model-path", "m", "--max-running-prompts", "0"]).output
    assert "--default-max-tokens must be positive" in runner.invoke(
        serve.serve_command, ["--model-path", "m", "--default-max-tokens", "0"]).output
    assert runner.invoke(serve.serve_command, []).exit_code != 0              # --model-path is required
    started = {}
    monkeypatch.setattr(serve, "create_app", lambda **kw: started.update(kw) or "app")
    monkeypatch.setattr("uvicorn.run", lambda app, host, port: started.update(app=app, host=host, port=port))
    monkeypatch.setattr("areno_b200.cli.model_refs.resolve_model_path", lambda p: f"resolved/{p}")
    res = runner.invoke(serve.serve_command, ["--model-path", "m", "--port", "9001", "--disable-thinking", "--kv-dtype", "fp8"])
    assert res.exit_code == 0, res.output
    assert started["model_path"] == "resolved/m" and started["port"] == 9001 and started["app"] == "app"
    assert started["chat_template_enable_thinking"] is False and started["kv_dtype"] == "fp8"


def test_request_defaults_match_the_sampling_defaults():
    req = serve.ChatCompletionRequest(messages=[serve.ChatMessage(role="user", content="x")])
    assert (req.temperature, req.top_p, req.top_k, req.n, req.stream, req.seed) == (1.0, 1.0, -1, 1, False, None)
    assert req.max_tokens is None and req.max_completion_tokens is None and req.stop is None and req.tools is None
    for bad in (dict(n=0), dict(max_tokens=0), dict(temperature=-0.1), dict(top_k=-2), dict(top_p=1.5)):
        with pytest.raises(Exception):
            serve.ChatCompletionRequest(messages=[], **bad)


def test_templates_receive_tools_tool_messages_and_flattened_content():
    tok = TemplateTokenizer()
    eng = ScriptedEngine(tok.encode("fine"))
    tools = [{"type": "function", "function": {"name": "look", "parameters": {"type": "object", "properties": {}}}}]
    app = serve.create_app(model_path="fake", engine=eng, tokenizer=tok)
    msgs = [{"role": "user", "content": [{"type": "text", "text": "see "}, {"type": "text", "text": "this"}]},
            {"role": "assistant", "content": None, "tool_calls": [{"id": "c", "type": "function",
                                                                   "function": {"name": "look", "arguments": "{}"}}]},
            {"role": "tool", "tool_call_id": "c", "name": "look", "content": "seen"}]
    with TestClient(app) as client:
        r = client.post("/v1/chat/completions", json={"messages": msgs, "tools": tools, "model": "alias"})
        assert r.status_code == 200 and r.json()["model"] == "alias"
    call = tok.calls[0]
    assert call["tools"] == tools
    assert [m["content"] for m in call["messages"]] == ["see this", "", "seen"]
    assert call["messages"][1]["tool_calls"][0]["function"]["arguments"] == {}     # a mapping, as templates expect
    assert call["messages"][2]["tool_call_id"] == "c" and call["messages"][2]["name"] == "look"
    prompts, _ = eng.calls[0]
    assert prompts[0] == tok.encode("[user] see this [assistant]  [tool] seen [assistant]")


def test_the_thinking_switch_reaches_the_template():
    tok = TemplateTokenizer()
    app = serve.create_app(model_path="fake", engine=ScriptedEngine([5]), tokenizer=tok,
                           chat_template_enable_thinking=False)
    with TestClient(app) as client:
        client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]})
    assert tok.calls[0]["enable_thinking"] is False


def test_stop_ids_come_from_eos_and_the_known_end_of_turn_tokens():
    vocab = {"<|im_end|>": 31, "<|eot_id|>": 2, "<|endoftext|>": 0, "<end_of_turn>": -1}

    class Tok:
        eos_token_id = [2, 9]
        unk_token_id = 0

        def convert_tokens_to_ids(self, t):
            if t == "<end_of_turn>":
                raise KeyError(t)
            return vocab[t]

    assert serve.stop_token_ids(Tok()) == (2, 9, 31)                 # no duplicate, no unknown id, no failing lookup
    assert serve.first_eos_token_id(Tok()) == 2
    assert serve.first_eos_token_id(SimpleNamespace(eos_token_id=[])) is None
    assert serve.first_eos_token_id(SimpleNamespace()) is None and serve.stop_token_ids(SimpleNamespace()) == ()


def test_prompts_beyond_the_context_are_refused_and_engine_failures_are_reported():
    tok = FakeTokenizer()
    eng = ScriptedEngine([5])
    eng.config.model.max_position_embeddings = 4
    app = serve.create_app(model_path="fake", engine=eng, tokenizer=tok)
    with TestClient(app, raise_server_exceptions=False) as client:
        r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a b c d e"}]})
        assert r.status_code == 400 and "model context is 4" in r.json()["detail"] and eng.calls == []

        async def boom(prompts, **kw):
            raise RuntimeError("engine fell over")

        eng.generate_rollout_async = boom
        r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a"}]})
        assert r.status_code == 500
        app.state.areno_serve.closing = True
        r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a"}]})
        assert r.status_code == 503 and "shutting down" in r.json()["detail"]
    assert eng.events == ["begin", "end", "close"]


def test_a_session_that_cannot_start_closes_the_engine():
    eng = ScriptedEngine([5])

    async def refuse():
        raise RuntimeError("no GPU")

    eng.begin_rollout_session_async = refuse
    app = serve.create_app(model_path="fake", engine=eng, tokenizer=FakeTokenizer())
    with pytest.raises(RuntimeError, match="no GPU"):
        with TestClient(app):
            pass
    assert eng.events == ["close"]


def test_choices_of_one_request_share_the_prompt_and_count_it_once_each():
    tok = FakeTokenizer()
    eng = ScriptedEngine(tok.encode("a b c"))
    app = serve.create_app(model_path="fake", engine=eng, tokenizer=tok, max_running_prompts=2)
    with TestClient(app) as client:
        body = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x y"}], "n": 3,
                                                         "max_tokens": 4, "top_k": 5}).json()
    assert [c["index"] for c in body["choices"]] == [0, 1, 2]
    assert body["usage"] == {"prompt_tokens": 6, "completion_tokens": 9, "total_tokens": 15}
    prompts, kw = eng.calls[0]
    assert prompts[0] == prompts[1] == prompts[2] and kw["max_running_prompts"] == 3     # never below the request's n
    assert kw["sampling_params"].top_k == 5 and kw["max_prompt_len"] == 256 - 4


def test_log_probabilities_of_the_sampled_tokens_on_request():
    tok = FakeTokenizer()
    ids = tok.encode("a b")
    eng = ScriptedEngine(ids)
    app = serve.create_app(model_path="fake", engine=eng, tokenizer=tok)
    with TestClient(app) as client:
        plain = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]}).json()
        assert plain["choices"][0]["logprobs"] is None
        body = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "logprobs": True,
                                                         "n": 2}).json()
    for choice in body["choices"]:
        content = choice["logprobs"]["content"]
        assert [c["token"] for c in content] == ["a", "b"] and [c["logprob"] for c in content] == [0.0, 0.0]
        assert all(c["top_logprobs"] == [] and c["bytes"] is None for c in content)
