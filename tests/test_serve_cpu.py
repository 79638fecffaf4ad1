"""OpenAI-compatible server over a tiny in-process CPU engine, and over a scripted fake engine for
the cancellation / tool-call paths."""

from __future__ import annotations

import asyncio
from types import SimpleNamespace

import pytest
from fastapi.testclient import TestClient

from areno_b200.cli import serve
from areno_b200.engine.inference import RolloutOutput

from .helpers import FakeTokenizer, write_tiny_checkpoint


class ScriptedEngine:
    """Returns fixed token ids; records what it was asked."""

    def __init__(self, ids, delay=0.0):
        self.ids, self.delay, self.calls, self.events = ids, delay, [], []
        self.config = SimpleNamespace(model=SimpleNamespace(max_position_embeddings=256))

    async def begin_rollout_session_async(self):
        self.events.append("begin")

    async def end_rollout_session_async(self):
        self.events.append("end")

    def close(self):
        self.events.append("close")

    async def generate_rollout_async(self, prompts, **kw):
        self.calls.append((prompts, kw))
        if self.delay:
            await asyncio.sleep(self.delay)
        n = len(prompts)
        return RolloutOutput(tokens=[list(self.ids) for _ in range(n)], logprobs=[[0.0] * len(self.ids)] * n,
                             finish_reasons=["stop"] * n, prompt_indices=list(range(n)))


def test_routes_with_scripted_engine():
    tok = FakeTokenizer()
    hello = tok.encode("hello world")
    eng = ScriptedEngine(hello)
    app = serve.create_app(model_path="fake-model", engine=eng, tokenizer=tok, default_max_tokens=7)
    with TestClient(app) as client:
        assert client.get("/health").json() == {"status": "ok"}
        assert client.get("/v1/models").json()["data"][0]["id"] == "fake-model"
        r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi there"}], "n": 2,
                                                      "temperature": 0.5, "seed": 3})
        assert r.status_code == 200, r.text
        body = r.json()
        assert [c["message"]["content"] for c in body["choices"]] == ["hello world"] * 2
        assert body["usage"]["completion_tokens"] == 2 * len(hello) and body["choices"][0]["finish_reason"] == "stop"
        prompts, kw = eng.calls[-1]
        assert len(prompts) == 2 and kw["max_new_tokens"] == 7 and kw["sampling_params"].temperature == 0.5
        assert kw["sampling_params"].seed == 3 and kw["eos_token_id"] == 2
        assert client.post("/v1/chat/completions", json={"messages": [], "n": 1}).status_code == 400
        assert client.post("/v1/chat/completions",
                           json={"messages": [{"role": "user", "content": "x"}], "stream": True}).status_code == 400
        assert client.post("/v1/chat/completions",
                           json={"messages": [{"role": "user", "content": "x"}], "top_p": 2.0}).status_code == 422
        r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "stop": ["world"],
                                                      "max_completion_tokens": 5})
        assert r.json()["choices"][0]["message"]["content"].strip() == "hello" and eng.calls[-1][1]["max_new_tokens"] == 5
    assert eng.events == ["begin", "end", "close"]


def test_tool_calls_are_parsed():
    tok = FakeTokenizer()
    text = '<tool_call> {"name":"get_weather","arguments":{"city":"Paris"}} </tool_call>'
    eng = ScriptedEngine(tok.encode(text))
    app = serve.create_app(model_path="qwen-fake", engine=eng, tokenizer=tok)
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}}}}}]
    with TestClient(app) as client:
        r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "weather?"}], "tools": tools})
        choice = r.json()["choices"][0]
        assert choice["finish_reason"] == "tool_calls"
        assert choice["message"]["tool_calls"][0]["function"]["name"] == "get_weather"


def test_disconnect_gives_cancelled_response():
    tok = FakeTokenizer()
    eng = ScriptedEngine(tok.encode("late"), delay=0.5)
    app = serve.create_app(model_path="fake", engine=eng, tokenizer=tok)
    state = app.state.areno_serve

    class GoneRequest:
        async def is_disconnected(self):
            return True

    async def scenario():
        req = serve.ChatCompletionRequest(messages=[serve.ChatMessage(role="user", content="x")], n=2)
        item = serve.PendingRequest(request=req, prompt=[5, 6], key=serve.BatchKey(4, 1.0, 1.0, -1, None, (2,), 2),
                                    future=asyncio.get_running_loop().create_future())
        task = asyncio.create_task(serve.run_request_task(state, item))
        resp = await serve.await_pending_response(state, GoneRequest(), item)
        await task
        return item, resp

    item, resp = asyncio.run(scenario())
    assert item.cancelled and len(resp.choices) == 2 and resp.usage.completion_tokens == 0
    assert all(c.finish_reason == "stop" for c in resp.choices)


def test_message_helpers():
    assert serve.message_content_text([{"type": "text", "text": "a"}, "b", {"type": "image_url", "image_url": "u"}]) == "ab"
    assert serve.normalize_stop("x") == ["x"] and serve.normalize_stop(["", "y"]) == ["y"] and serve.normalize_stop(None) == []
    assert serve.stop_token_ids(FakeTokenizer()) == (2,) and serve.first_eos_token_id(FakeTokenizer()) == 2
    with pytest.raises(ValueError):
        serve.create_app(model_path="m", world_size=3, tp_size=2, engine=object(), tokenizer=FakeTokenizer())


def test_real_engine_roundtrip(tmp_path):
    """HTTP request -> tokenizer -> in-process engine (CPU reference kernels) -> decoded completion."""
    from areno_b200.engine.api import ArenoEngine
    from areno_b200.engine.config import RuntimeConfig

    path = str(tmp_path / "ckpt")
    write_tiny_checkpoint(path)
    eng = ArenoEngine.from_pretrained(path, tp_size=1, dp_size=1, runtime_config=RuntimeConfig(eager_decode=True),
                                      loss_fn=serve.serve_loss_fn, launcher="inprocess", max_running_seqs=4)
    app = serve.create_app(model_path=path, engine=eng, tokenizer=FakeTokenizer(), default_max_tokens=6)
    with TestClient(app) as client:
        payload = {"messages": [{"role": "user", "content": "one two three"}], "n": 2, "seed": 11, "temperature": 1.0}
        a = client.post("/v1/chat/completions", json=payload).json()
        b = client.post("/v1/chat/completions", json=payload).json()
        assert a["usage"]["completion_tokens"] >= 2 and len(a["choices"]) == 2
        assert 1 <= a["usage"]["completion_tokens"] <= 12
        assert [c["message"] for c in a["choices"]] == [c["message"] for c in b["choices"]]  # seeded
