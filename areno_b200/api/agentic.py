"""Agentic rollouts: a rollout session with a local OpenAI-compatible proxy.

Agent code receives a ``RolloutSession`` and an ``AgentBatch``; it talks to
``session.get_base_url()`` with any OpenAI client (``POST /v1/chat/completions``, non-streaming)
and returns an ``AgentTrajectory`` whose turns hold the request messages and the raw proxy
responses.  Each response carries an ``areno`` block with the exact prompt / response token ids
and rollout log-probs, so training rows are rebuilt from tokens, never by re-tokenising text.
Turns of one (prompt, sample) pair are merged into a single training row by extending the
previous row past their common token prefix; which spans contribute to the loss is decided by
``LossMaskPolicy`` (tool results echoed after a generated tool call are always masked).

Public names and semantics follow ``areno/api/agentic.py:46-998`` of the reference; the merge logic
lives in ``SampleAccumulator`` instead of private session methods called by trainers.
"""

from __future__ import annotations

import asyncio
import importlib.util
import json
import threading
import time
import uuid
from collections.abc import Callable, Iterator
from dataclasses import dataclass, field
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path
from typing import Any

from ..utils.log import get_logger
from .openai_chat import (build_chat_completion_response, first_user_text, messages_to_prompt_tokens, messages_to_text,
                          normalize_messages)
from .rewards import RewardEvent, RewardRecord
from .tokenizer import apply_chat_template_with_options
from .tool_call_parser import get_tool_call_parser, infer_tool_call_parser_name

logger = get_logger("agentic")


# ------------------------------------------------------------------------ data model
@dataclass
class LossMaskPolicy:
    assistant_text: bool = True
    assistant_tool_calls: bool = True
    tool_results: bool = False
    final_assistant_text: bool = True
    system_prompt: bool = False
    user_prompt: bool = False

    def span_enabled(self, kind: str) -> bool:
        return self.assistant_tool_calls if kind == "assistant_tool_call" else self.assistant_text


@dataclass
class AgentItem:
    record: dict[str, Any]
    prompt: str
    input_tokens: list[int]
    prompt_index: int
    sample_index: int


@dataclass
class AgentBatch:
    records: list[dict[str, Any]]
    prompts: list[str]
    input_tokens: list[list[int]]
    n_samples: int

    def __len__(self) -> int:
        return len(self.records) * self.n_samples

    @classmethod
    def from_prompt_batch(cls, prompt_batch, n_samples: int) -> "AgentBatch":
        return cls(records=[dict(i.record) for i in prompt_batch.items], prompts=[i.prompt for i in prompt_batch.items],
                   input_tokens=[list(i.input_tokens) for i in prompt_batch.items], n_samples=int(n_samples))

    def iter_samples(self) -> Iterator[AgentItem]:
        for pi, (rec, prompt, toks) in enumerate(zip(self.records, self.prompts, self.input_tokens)):
            for si in range(self.n_samples):
                yield AgentItem(record=rec, prompt=prompt, input_tokens=toks, prompt_index=pi, sample_index=si)


@dataclass
class AgentTrainBatch:
    token_rows: list[list[int]]
    response_masks: list[list[bool]]
    loss_masks: list[list[bool]]
    rollout_logprobs: list[list[float]]
    rewards: list[float] | None
    records: list[dict[str, Any]]
    reward_records: list[RewardRecord]


def _get(obj: Any, key: str) -> Any:
    return obj.get(key) if isinstance(obj, dict) else getattr(obj, key, None)


def response_areno_metadata(response: Any) -> dict[str, Any]:
    """The ``areno`` block of a proxy response (dict or OpenAI client object)."""
    meta = None
    if isinstance(response, dict):
        meta = response.get("areno")
    else:
        extra = getattr(response, "model_extra", None)
        if isinstance(extra, dict):
            meta = extra.get("areno")
        if meta is None:
            meta = getattr(response, "areno", None)
    if not isinstance(meta, dict):
        raise ValueError("chat response does not include Areno trajectory metadata")
    toks, lps = meta.get("response_tokens"), meta.get("response_logprobs")
    if not isinstance(toks, list) or not isinstance(lps, list):
        raise ValueError("Areno trajectory metadata must include response_tokens and response_logprobs lists")
    if len(toks) != len(lps):
        raise ValueError("Areno trajectory metadata response_tokens/response_logprobs length mismatch")
    return meta


def response_tool_calls(response: Any) -> list[dict[str, Any]]:
    """Tool calls as parsed by the proxy (agents never re-parse model text)."""
    choices = _get(response, "choices")
    if not isinstance(choices, list) or not choices:
        return []
    raw = _get(_get(choices[0], "message") or {}, "tool_calls")
    calls = []
    for c in raw if isinstance(raw, list) else []:
        fn = _get(c, "function") or {}
        name = _get(fn, "name")
        if not name:
            continue
        args = _get(fn, "arguments")
        if not isinstance(args, str):
            args = json.dumps(args if args is not None else {}, ensure_ascii=False, sort_keys=True)
        calls.append({"id": _get(c, "id") or f"call_{uuid.uuid4().hex}", "type": _get(c, "type") or "function",
                      "function": {"name": str(name), "arguments": args}})
    return calls


@dataclass
class AgentTrajectoryTurn:
    item: AgentItem
    messages: list[dict[str, Any]]
    response: Any | None = None
    response_tokens: list[int] = field(default_factory=list)
    response_logprobs: list[float] = field(default_factory=list)
    parsed_tool_calls: list[dict[str, Any]] = field(default_factory=list)
    model: str = "policy"
    tools: list[dict[str, Any]] = field(default_factory=list)
    tool_choice: Any = None

    def __post_init__(self) -> None:
        if self.response is None:
            return
        meta = response_areno_metadata(self.response)
        self.response_tokens = list(meta["response_tokens"])
        self.response_logprobs = [float(v) for v in meta["response_logprobs"]]
        self.parsed_tool_calls = response_tool_calls(self.response)


@dataclass
class AgentTrajectory:
    turns: list[AgentTrajectoryTurn] = field(default_factory=list)


# ------------------------------------------------------------------ row accumulation
def common_prefix_len(a: list[int], b: list[int]) -> int:
    n = min(len(a), len(b))
    for i in range(n):
        if a[i] != b[i]:
            return i
    return n


def tool_call_loss_mask(tokenizer, response_tokens: list[int]) -> list[bool]:
    """All True up to a tool-response sentinel echoed inside a generated tool call, False after."""
    mask = [True] * len(response_tokens)
    try:
        text = tokenizer.decode(response_tokens)
    except Exception:
        return mask
    cut = min((p for p in (text.find(m) for m in ("<|tool_response>", "<tool_response>")) if p >= 0), default=-1)
    if cut < 0:
        return mask
    try:
        keep = len(tokenizer.encode(text[:cut]))
    except Exception:
        return mask
    for i in range(min(keep, len(mask)), len(mask)):
        mask[i] = False
    return mask


@dataclass
class AgentSample:
    """Everything known about one (prompt, sample) pair after merging its turns."""

    item: AgentItem
    messages: list[dict[str, Any]]
    response_text: str
    last_response_text: str
    response_tokens: list[int]
    response_logprobs: list[float]
    response_loss_mask: list[bool]
    trace: list[RewardEvent]
    last_tool_calls: list[dict[str, Any]] = field(default_factory=list)
    token_row: list[int] = field(default_factory=list)
    response_mask_row: list[bool] = field(default_factory=list)
    loss_mask_row: list[bool] = field(default_factory=list)
    rollout_logprobs_row: list[float] = field(default_factory=list)


class SampleAccumulator:
    """Builds ``AgentSample`` objects from trajectory turns, merging turns of the same pair."""

    def __init__(self, tokenizer, policy: LossMaskPolicy):
        self.tokenizer = tokenizer
        self.policy = policy
        self.samples: list[AgentSample] = []
        self._index: dict[tuple[int, int], AgentSample] = {}

    def _turn_sample(self, turn: AgentTrajectoryTurn) -> AgentSample:
        messages = normalize_messages(turn.messages)
        prompt_tokens = messages_to_prompt_tokens(self.tokenizer, messages, tools=turn.tools,
                                                  fallback_prompt=turn.item.prompt)
        text = self.tokenizer.decode(turn.response_tokens)
        calls = list(turn.parsed_tool_calls or [])
        kind = "assistant_tool_call" if calls else "assistant_text"
        if calls:
            events = [RewardEvent(type="assistant_tool_call", name=c["function"]["name"],
                                  arguments=c["function"]["arguments"]) for c in calls]
            mask = tool_call_loss_mask(self.tokenizer, turn.response_tokens)
            if not self.policy.span_enabled(kind):
                mask = [False] * len(mask)
        else:
            events = [RewardEvent(type=kind, text=text)]
            mask = [self.policy.span_enabled(kind)] * len(turn.response_tokens)
        trace = [RewardEvent(type="request", messages=messages), *events,
                 RewardEvent(type="finish", metadata={"finish_reason": "stop"})]
        n_p, n_r = len(prompt_tokens), len(turn.response_tokens)
        return AgentSample(
            item=turn.item, messages=messages, response_text=text, last_response_text=text,
            response_tokens=list(turn.response_tokens), response_logprobs=list(turn.response_logprobs),
            response_loss_mask=mask, trace=trace, last_tool_calls=calls,
            token_row=list(prompt_tokens) + list(turn.response_tokens),
            response_mask_row=[False] * n_p + [True] * n_r, loss_mask_row=[False] * n_p + list(mask),
            rollout_logprobs_row=[0.0] * n_p + list(turn.response_logprobs))

    def add_turn(self, turn: AgentTrajectoryTurn) -> AgentSample:
        new = self._turn_sample(turn)
        key = (turn.item.prompt_index, turn.item.sample_index)
        cur = self._index.get(key)
        if cur is None:
            self._index[key] = new
            self.samples.append(new)
            return new
        if new.response_text:
            cur.response_text = f"{cur.response_text}\n{new.response_text}" if cur.response_text else new.response_text
            cur.last_response_text = new.response_text
            cur.last_tool_calls = list(new.last_tool_calls)
        cur.response_tokens.extend(new.response_tokens)
        cur.response_logprobs.extend(new.response_logprobs)
        cur.response_loss_mask.extend(new.response_loss_mask)
        cur.trace.extend(new.trace)
        cur.messages = new.messages
        # the new turn's prompt re-renders the whole conversation: keep the shared prefix, append the rest
        keep = common_prefix_len(cur.token_row, new.token_row)
        if keep < len(new.token_row):
            cur.token_row.extend(new.token_row[keep:])
            cur.response_mask_row.extend(new.response_mask_row[keep:])
            cur.loss_mask_row.extend(new.loss_mask_row[keep:])
            cur.rollout_logprobs_row.extend(new.rollout_logprobs_row[keep:])
        return cur


def tool_results_from_messages(messages: list[dict[str, Any]]) -> list[dict[str, Any]]:
    return [{"name": m.get("name"), "tool_call_id": m.get("tool_call_id"), "content": m.get("content")}
            for m in messages if m.get("role") == "tool"]


def render_messages(tokenizer, messages: list[dict[str, Any]]) -> str:
    messages = normalize_messages(messages)
    if getattr(tokenizer, "chat_template", None):
        try:
            out = apply_chat_template_with_options(tokenizer, messages, tokenize=False, add_generation_prompt=False)
            if isinstance(out, str):
                return out
        except Exception:
            pass
    return messages_to_text(messages)


def _max_context_len(params: Any) -> int | None:
    for attr in ("max_context_len", "max_prompt_len"):
        v = getattr(params, attr, None)
        if v is not None:
            return int(v)
    return None


# -------------------------------------------------------------------------- session
class _ProxyServer(ThreadingHTTPServer):
    daemon_threads = True
    request_queue_size = 2048

    def __init__(self, *args, max_threads: int = 2048, **kwargs):
        super().__init__(*args, **kwargs)
        self._slots = threading.BoundedSemaphore(max_threads)

    def process_request(self, request, client_address):
        self._slots.acquire()
        try:
            super().process_request(request, client_address)
        except BaseException:
            self._slots.release()
            raise

    def process_request_thread(self, request, client_address):
        try:
            super().process_request_thread(request, client_address)
        finally:
            self._slots.release()


def _write_json(handler: BaseHTTPRequestHandler, status: int, payload: dict[str, Any]) -> None:
    data = json.dumps(payload).encode("utf-8")
    try:
        handler.send_response(status)
        handler.send_header("content-type", "application/json")
        handler.send_header("content-length", str(len(data)))
        handler.end_headers()
        handler.wfile.write(data)
    except (BrokenPipeError, ConnectionAbortedError, ConnectionResetError):
        logger.debug("agentic proxy client disconnected before response write")


class RolloutSession:
    """Rollout session: ``with`` for plain batched rollouts, ``async with`` for agentic rollouts behind
    the local proxy (``http://127.0.0.1:<port>/v1``)."""

    api_key = "areno-agentic"

    def __init__(self, trainer, *, sampling_params, loss_mask_policy: LossMaskPolicy | None = None,
                 max_running_prompts: int | None = None, timeout_s: float = 300.0, proxy: bool = True) -> None:
        self._trainer = trainer
        self._sampling_params = sampling_params
        self._policy = loss_mask_policy or LossMaskPolicy()
        self._parser = get_tool_call_parser(infer_tool_call_parser_name(trainer))
        try:
            self._dp = max(int(trainer.dp_size()), 1)
        except Exception:
            self._dp = 1
        self._max_running = max(1, int(max_running_prompts)) if max_running_prompts is not None else self._dp
        self._timeout_s = float(timeout_s)
        self._proxy_enabled = bool(proxy)
        self._server: ThreadingHTTPServer | None = None
        self._thread: threading.Thread | None = None
        self._loop: asyncio.AbstractEventLoop | None = None
        self._base_url = ""

    # plain (synchronous) use
    def __enter__(self) -> "RolloutSession":
        self._trainer.begin_rollout_session()
        return self

    def __exit__(self, *_exc) -> None:
        self._trainer.end_rollout_session()

    # agentic (asynchronous) use
    async def __aenter__(self) -> "RolloutSession":
        self._loop = asyncio.get_running_loop()
        await self._trainer.begin_rollout_session_async()
        if not self._proxy_enabled:
            return self
        session = self

        class Handler(BaseHTTPRequestHandler):
            def do_POST(self):  # noqa: N802
                session._handle_post(self)

            def log_message(self, fmt, *args):
                pass

        try:
            self._server = _ProxyServer(("127.0.0.1", 0), Handler)
            self._server.timeout = 0.5
            host, port = self._server.server_address[:2]
            self._base_url = f"http://{host}:{port}/v1"
            self._thread = threading.Thread(target=self._server.serve_forever, name="areno-agentic-proxy", daemon=True)
            self._thread.start()
        except BaseException:
            await self._trainer.end_rollout_session_async()
            raise
        return self

    async def __aexit__(self, *_exc) -> None:
        try:
            if self._server is not None:
                self._server.shutdown()
                self._server.server_close()
            if self._thread is not None:
                self._thread.join(timeout=2.0)
        finally:
            await self._trainer.end_rollout_session_async()

    @property
    def max_running_prompts(self) -> int:
        return self._max_running

    @property
    def base_url(self) -> str:
        if not self._proxy_enabled:
            raise RuntimeError("rollout session proxy is disabled")
        return self._base_url

    def get_base_url(self) -> str:
        return self.base_url

    def finish_requests(self) -> None:
        """Kept for agents that signal the end of request submission; nothing to do."""

    async def sync_rollout_session_async(self) -> None:
        await self._trainer.sync_rollout_session_async()

    # ------------------------------------------------------------------ proxy
    def _handle_post(self, handler: BaseHTTPRequestHandler) -> None:
        if handler.path not in {"/v1/chat/completions", "/chat/completions"}:
            _write_json(handler, 404, {"error": {"message": f"unsupported path: {handler.path}"}})
            return
        try:
            body = json.loads(handler.rfile.read(int(handler.headers.get("content-length", "0"))).decode("utf-8") or "{}")
        except json.JSONDecodeError as exc:
            _write_json(handler, 400, {"error": {"message": f"invalid json: {exc}"}})
            return
        if body.get("stream"):
            _write_json(handler, 400, {"error": {"message": "streaming chat completions are not supported yet"}})
            return
        if self._loop is None:
            _write_json(handler, 500, {"error": {"message": "agent rollout proxy is not running"}})
            return
        try:
            fut = asyncio.run_coroutine_threadsafe(self.complete_chat(body), self._loop)
            _write_json(handler, 200, fut.result(timeout=self._timeout_s))
        except ValueError as exc:
            _write_json(handler, 400, {"error": {"message": str(exc)}})
        except Exception as exc:  # noqa: BLE001
            _write_json(handler, 500, {"error": {"message": str(exc) or type(exc).__name__}})

    async def complete_chat(self, body: dict[str, Any]) -> dict[str, Any]:
        """One chat completion through the trainer's async rollout path."""
        messages = normalize_messages(body.get("messages") or [])
        if not messages:
            raise ValueError("messages must be non-empty")
        tools = list(body.get("tools") or [])
        tool_choice = body.get("tool_choice")
        params = self._sampling_params.model_copy() if hasattr(self._sampling_params, "model_copy") \
            else self._sampling_params.copy()
        if body.get("max_tokens") is not None:
            params.max_new_tokens = int(body["max_tokens"])
        if body.get("temperature") is not None:
            params.temperature = float(body["temperature"])
        if body.get("top_p") is not None:
            params.top_p = float(body["top_p"])
        model = body.get("model") or "policy"
        tokenizer = self._trainer.get_tokenizer()
        input_tokens = messages_to_prompt_tokens(tokenizer, messages, tools=tools,
                                                 fallback_prompt=first_user_text(messages))
        limit = _max_context_len(params)
        if limit is not None and len(input_tokens) > limit:
            return {"id": f"chatcmpl-{uuid.uuid4().hex}", "object": "chat.completion", "created": int(time.time()),
                    "model": model,
                    "choices": [{"index": 0, "message": {"role": "assistant", "content": ""}, "finish_reason": "length"}],
                    "usage": {"prompt_tokens": len(input_tokens), "completion_tokens": 0,
                              "total_tokens": len(input_tokens), "max_sequence_len": limit},
                    "areno": {"input_tokens": [], "response_tokens": [], "response_logprobs": []}}
        try:
            results = await asyncio.wait_for(
                self._trainer.rollout_token_batch_async([input_tokens], 1, params), timeout=self._timeout_s)
        except asyncio.TimeoutError:
            raise TimeoutError("agent rollout proxy timed out waiting for completion") from None
        seq = results[0].sequences[0] if results and results[0].sequences else None
        toks = list(seq.resp_tokens) if seq is not None else []
        lps = list(seq.resp_logprobs) if seq is not None else []
        content = tokenizer.decode(toks)
        calls = self._parser.parse(content, tools, tool_choice).tool_calls
        return build_chat_completion_response(
            tokenizer=tokenizer, model=model, prompt_tokens=len(input_tokens), response_ids=[toks],
            finish_reasons=["tool_calls" if calls else "stop"], tools=tools, tool_choice=tool_choice,
            tool_call_parser=self._parser, parsed_tool_calls=[calls], response_logprobs=[lps],
            include_areno_metadata=True, input_tokens=input_tokens)

    # ------------------------------------------------------- trajectories -> batch
    def accumulate(self, trajectories) -> list[AgentSample]:
        """Merge the turns of one or more ``AgentTrajectory`` objects into per-pair samples."""
        acc = SampleAccumulator(self._trainer.get_tokenizer(), self._policy)
        trajs = trajectories if isinstance(trajectories, (list, tuple)) else [trajectories]
        for traj in trajs:
            for turn in (traj.turns if isinstance(traj, AgentTrajectory) else traj):
                acc.add_turn(turn)
        return acc.samples

    def reward_record(self, sample: AgentSample) -> RewardRecord:
        answer = sample.item.record.get("answer", sample.item.record.get("solutions"))
        messages = list(sample.messages)
        if sample.last_tool_calls:
            messages.append({"role": "assistant", "content": "", "tool_calls": list(sample.last_tool_calls)})
        else:
            messages.append({"role": "assistant", "content": sample.last_response_text})
        results = tool_results_from_messages(messages)
        trace = list(sample.trace)
        if results:
            events = [RewardEvent(type="tool_result", name=r.get("name"), content=r.get("content"),
                                  metadata={"tool_call_id": r["tool_call_id"]} if r.get("tool_call_id") is not None else {})
                      for r in results]
            pos = next((i for i, e in enumerate(trace) if e.type == "finish"), len(trace))
            trace[pos:pos] = events
        return RewardRecord(
            prompt=sample.item.prompt, completion=sample.response_text,
            rendered_completion=render_messages(self._trainer.get_tokenizer(), messages),
            final_answer=sample.last_response_text, answer=answer, messages=messages, trace=trace,
            tool_calls=[{"name": e.name, "arguments": e.arguments} for e in sample.trace
                        if e.type == "assistant_tool_call" and e.name is not None],
            tool_results=results, tokens=sample.response_tokens, logprobs=sample.response_logprobs,
            loss_mask=list(sample.response_loss_mask), source_record=sample.item.record,
            metadata={"prompt_index": sample.item.prompt_index, "sample_index": sample.item.sample_index})

    def build_train_batch(self, samples: list[AgentSample], reward_fn: Callable[[RewardRecord], float] | None
                          ) -> AgentTrainBatch:
        records = [self.reward_record(s) for s in samples]
        rewards = [float(reward_fn(r)) for r in records] if reward_fn is not None else None
        return AgentTrainBatch(
            token_rows=[list(s.token_row) for s in samples], response_masks=[list(s.response_mask_row) for s in samples],
            loss_masks=[list(s.loss_mask_row) for s in samples],
            rollout_logprobs=[list(s.rollout_logprobs_row) for s in samples], rewards=rewards,
            records=[s.item.record for s in samples], reward_records=records)


def load_agent_run_fn(path: str) -> Callable[[RolloutSession, AgentBatch], Any]:
    """Load ``run_agent(session, batch)`` (sync or async) from a Python file."""
    module_path = Path(path).expanduser().resolve()
    spec = importlib.util.spec_from_file_location(module_path.stem, module_path)
    if spec is None or spec.loader is None:
        raise ValueError(f"cannot load agent function from {module_path}")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    fn = getattr(module, "run_agent", None)
    if not callable(fn):
        raise ValueError(f"{module_path} must define callable run_agent(ctx, batch)")
    return fn


async def maybe_await(value):
    if asyncio.iscoroutine(value) or isinstance(value, asyncio.Future):
        return await value
    return value
