"""``areno serve``: an OpenAI-compatible chat-completions server on top of ``ArenoEngine``.

Routes: ``GET /health``, ``GET /v1/models``, ``POST /v1/chat/completions`` (non-streaming; ``n``
completions, ``tools`` / ``tool_choice`` with a model-specific tool-call parser, ``stop`` strings,
``seed``).  One rollout session stays open for the life of the server; every HTTP request becomes an
independent ``generate_rollout_async`` call that joins the running batch of one data-parallel row
(continuous batching happens in the worker loop, not here).  A watcher polls the connection: when a
client goes away its request is answered with an empty ``stop`` completion and the engine call is
left to drain.  Same surface as ``areno/cli/serve.py:41-597`` in the reference.
"""

from __future__ import annotations

import asyncio
import time
from contextlib import asynccontextmanager
from dataclasses import dataclass, field
from typing import Any, Literal

import click
from fastapi import FastAPI, HTTPException, Request
from pydantic import BaseModel, Field

DISCONNECT_POLL_S = 0.1


def serve_loss_fn(*_: Any):
    raise RuntimeError("the serving engine does not support training")


class ChatMessage(BaseModel):
    role: Literal["system", "user", "assistant", "tool"] | str
    content: str | list[Any] | None = None
    name: str | None = None
    tool_call_id: str | None = None
    tool_calls: list[dict[str, Any]] | None = None


class ChatCompletionRequest(BaseModel):
    model: str | None = None
    messages: list[ChatMessage]
    tools: list[dict[str, Any]] | None = None
    tool_choice: Any = None
    max_tokens: int | None = Field(default=None, ge=1)
    max_completion_tokens: int | None = Field(default=None, ge=1)
    temperature: float = Field(default=1.0, ge=0.0)
    top_p: float = Field(default=1.0, ge=0.0, le=1.0)
    top_k: int = Field(default=-1, ge=-1)
    n: int = Field(default=1, ge=1)
    stream: bool = False
    stop: str | list[str] | None = None
    seed: int | None = None
    logprobs: bool = False            # return the sampled tokens' log-probabilities (no top-k alternatives)


class ChatCompletionChoice(BaseModel):
    index: int
    message: dict[str, Any]
    finish_reason: str
    logprobs: dict[str, Any] | None = None


class ChatCompletionUsage(BaseModel):
    prompt_tokens: int
    completion_tokens: int
    total_tokens: int


class ChatCompletionResponse(BaseModel):
    id: str
    object: str = "chat.completion"
    created: int
    model: str
    choices: list[ChatCompletionChoice]
    usage: ChatCompletionUsage


@dataclass(frozen=True)
class BatchKey:
    """Everything that decides how a request is sampled."""

    max_new_tokens: int
    temperature: float
    top_p: float
    top_k: int
    seed: int | None
    stop_token_ids: tuple[int, ...]
    eos_token_id: int | None


@dataclass
class PendingRequest:
    request: ChatCompletionRequest
    prompt: list[int]
    key: BatchKey
    future: asyncio.Future
    created_at: float = field(default_factory=time.monotonic)
    cancelled: bool = False


@dataclass
class ServeState:
    model_path: str
    tokenizer: Any
    engine: Any
    max_running_prompts: int
    default_max_tokens: int
    max_model_len: int
    tool_call_parser: Any
    decode_progress_interval_s: float = 0.0
    active_tasks: set = field(default_factory=set)
    closing: bool = False
    session_open: bool = False


class _ParserProbe:
    """Gives ``infer_tool_call_parser_name`` the two things it reads: a tokenizer and a model path."""

    def __init__(self, model_path: str, tokenizer: Any):
        self._model_path = model_path
        self._tokenizer = tokenizer

    def get_tokenizer(self):
        return self._tokenizer


# --------------------------------------------------------------------- message helpers
def message_content_text(content: str | list[Any] | None) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    parts = []
    for piece in content:
        if isinstance(piece, str):
            parts.append(piece)
        elif isinstance(piece, dict):
            if piece.get("type") in (None, "text", "input_text") and isinstance(piece.get("text"), str):
                parts.append(piece["text"])
        elif hasattr(piece, "text") and isinstance(piece.text, str):
            parts.append(piece.text)
    return "".join(parts)


def chat_message_payload(message: ChatMessage) -> dict[str, Any]:
    out: dict[str, Any] = {"role": message.role, "content": message_content_text(message.content)}
    for name in ("name", "tool_call_id", "tool_calls"):
        value = getattr(message, name)
        if value is not None:
            out[name] = value
    return out


def encode_messages(tokenizer: Any, messages: list[ChatMessage], *, tools=None) -> list[int]:
    from ..api.openai_chat import messages_to_prompt_tokens

    payload = [chat_message_payload(m) for m in messages]
    fallback = "\n".join(f"{m['role']}: {m['content']}" for m in payload)
    return messages_to_prompt_tokens(tokenizer, payload, tools=tools, fallback_prompt=fallback)


def first_eos_token_id(tokenizer: Any) -> int | None:
    eos = getattr(tokenizer, "eos_token_id", None)
    if isinstance(eos, (list, tuple)):
        return int(eos[0]) if eos else None
    return int(eos) if eos is not None else None


def stop_token_ids(tokenizer: Any) -> tuple[int, ...]:
    ids: list[int] = []
    eos = getattr(tokenizer, "eos_token_id", None)
    for v in (eos if isinstance(eos, (list, tuple)) else [eos]):
        if v is not None and int(v) not in ids:
            ids.append(int(v))
    convert = getattr(tokenizer, "convert_tokens_to_ids", None)
    unk = getattr(tokenizer, "unk_token_id", None)
    if convert is not None:
        for tok in ("<|im_end|>", "<|eot_id|>", "<|endoftext|>", "<end_of_turn>"):
            try:
                v = convert(tok)
            except Exception:
                continue
            if isinstance(v, int) and v >= 0 and v != unk and v not in ids:
                ids.append(v)
    return tuple(ids)


def normalize_stop(stop: str | list[str] | None) -> list[str]:
    if stop is None:
        return []
    items = [stop] if isinstance(stop, str) else list(stop)
    return [s for s in items if isinstance(s, str) and s]


# ------------------------------------------------------------------- response building
def build_response(state: ServeState, request: ChatCompletionRequest, prompt: list[int],
                   response_ids: list[list[int]], finish_reasons: list[str],
                   response_logprobs: list[list[float]] | None = None) -> ChatCompletionResponse:
    from ..api.openai_chat import build_chat_completion_response

    data = build_chat_completion_response(
        tokenizer=state.tokenizer, model=request.model or state.model_path,
        prompt_tokens=len(prompt) * len(response_ids), response_ids=response_ids, finish_reasons=finish_reasons,
        tools=request.tools, tool_choice=request.tool_choice, tool_call_parser=state.tool_call_parser,
        stop_strings=normalize_stop(request.stop), response_logprobs=response_logprobs,
        include_logprobs=bool(request.logprobs))
    return ChatCompletionResponse(**data)


def cancelled_response(state: ServeState, item: PendingRequest) -> ChatCompletionResponse:
    n = int(item.request.n)
    return build_response(state, item.request, item.prompt, [[] for _ in range(n)], ["stop"] * n)


# ----------------------------------------------------------------------- request tasks
async def run_request_rollout(state: ServeState, item: PendingRequest) -> ChatCompletionResponse | None:
    from ..engine.inference import SamplingParams

    if item.cancelled or item.future.done():
        return None
    key = item.key
    prompts = [item.prompt for _ in range(int(item.request.n))]
    rollout = await state.engine.generate_rollout_async(
        prompts, max_new_tokens=key.max_new_tokens,
        max_running_prompts=max(state.max_running_prompts, len(prompts)),
        max_prompt_len=max(state.max_model_len - key.max_new_tokens, len(item.prompt)),
        eos_token_id=key.eos_token_id,
        sampling_params=SamplingParams(temperature=key.temperature, top_p=key.top_p, top_k=key.top_k, seed=key.seed,
                                       stop_token_ids=key.stop_token_ids),
        decode_progress_interval_s=state.decode_progress_interval_s)
    if item.future.done():
        return None
    return build_response(state, item.request, item.prompt, rollout.response_ids, rollout.finish_reason,
                          rollout.response_logprobs)


async def run_request_task(state: ServeState, item: PendingRequest) -> None:
    try:
        resp = await run_request_rollout(state, item)
        if resp is not None and not item.future.done():
            item.future.set_result(resp)
    except BaseException as exc:  # delivered to the awaiting handler
        if not item.future.done():
            item.future.set_exception(exc)


async def watch_disconnect(state: ServeState, raw_request, item: PendingRequest) -> None:
    while not item.future.done():
        if await raw_request.is_disconnected():
            item.cancelled = True
            if not item.future.done():
                item.future.set_result(cancelled_response(state, item))
            return
        await asyncio.sleep(DISCONNECT_POLL_S)


async def await_pending_response(state: ServeState, raw_request, item: PendingRequest) -> ChatCompletionResponse:
    watcher = asyncio.create_task(watch_disconnect(state, raw_request, item))
    try:
        # shield: a cancelled handler must not cancel the future other code resolves
        return await asyncio.shield(item.future)
    except asyncio.CancelledError:
        item.cancelled = True
        return cancelled_response(state, item)
    finally:
        watcher.cancel()


# --------------------------------------------------------------------------------- app
def create_app(*, model_path: str, tp_size: int = 1, world_size: int = 1, max_running_prompts: int = 64,
               default_max_tokens: int = 1024, decode_progress_interval_s: float = 0.0, eager_decode: bool = False,
               attn_backend: Literal["flash", "native"] = "flash", kv_dtype: str = "bf16",
               chat_template_enable_thinking: bool | None = None, engine: Any = None, tokenizer: Any = None):
    """Build the FastAPI app.  ``engine`` / ``tokenizer`` may be injected (tests, embedding in another
    process); otherwise the tokenizer is loaded from ``model_path`` and an engine is started on
    ``world_size`` local GPUs."""
    from ..api.tokenizer import configure_chat_template_enable_thinking, load_tokenizer
    from ..api.tool_call_parser import get_tool_call_parser, infer_tool_call_parser_name

    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    if tp_size < 1:
        raise ValueError("tp_size must be >= 1")
    if world_size % tp_size != 0:
        raise ValueError("world_size must be divisible by tp_size")
    if tokenizer is None:
        tokenizer = load_tokenizer(model_path)
    configure_chat_template_enable_thinking(tokenizer, chat_template_enable_thinking)
    if engine is None:
        from ..engine.api import ArenoEngine
        from ..engine.config import RuntimeConfig

        engine = ArenoEngine.from_pretrained(
            model_path, tp_size=tp_size, dp_size=world_size // tp_size, devices=list(range(world_size)),
            runtime_config=RuntimeConfig(eager_decode=bool(eager_decode), attn_backend=attn_backend, kv_dtype=kv_dtype),
            loss_fn=serve_loss_fn, max_running_seqs=max_running_prompts)
    model_cfg = getattr(getattr(engine, "config", None), "model", None)
    state = ServeState(
        model_path=model_path, tokenizer=tokenizer, engine=engine, max_running_prompts=max_running_prompts,
        default_max_tokens=default_max_tokens,
        max_model_len=int(getattr(model_cfg, "max_position_embeddings", 0) or 32768),
        tool_call_parser=get_tool_call_parser(infer_tool_call_parser_name(_ParserProbe(model_path, tokenizer))),
        decode_progress_interval_s=float(decode_progress_interval_s))

    @asynccontextmanager
    async def lifespan(_app):
        try:
            await state.engine.begin_rollout_session_async()
        except BaseException:
            state.engine.close()
            raise
        state.session_open = True
        try:
            yield
        finally:
            state.closing = True
            if state.active_tasks:
                await asyncio.gather(*state.active_tasks, return_exceptions=True)
            try:
                if state.session_open:
                    await state.engine.end_rollout_session_async()
            finally:
                state.engine.close()

    app = FastAPI(title="areno-b200 OpenAI-compatible server", lifespan=lifespan)
    app.state.areno_serve = state

    @app.get("/health")
    def health() -> dict[str, str]:
        return {"status": "ok"}

    @app.get("/v1/models")
    def models() -> dict[str, Any]:
        return {"object": "list",
                "data": [{"id": state.model_path, "object": "model", "created": 0, "owned_by": "areno"}]}

    @app.post("/v1/chat/completions", response_model=ChatCompletionResponse)
    async def chat_completions(raw_request: Request, request: ChatCompletionRequest) -> ChatCompletionResponse:
        if request.stream:
            raise HTTPException(status_code=400, detail="stream=true is not supported")
        if not request.messages:
            raise HTTPException(status_code=400, detail="messages must be non-empty")
        prompt = encode_messages(state.tokenizer, request.messages, tools=request.tools)
        key = BatchKey(
            max_new_tokens=int(request.max_completion_tokens or request.max_tokens or state.default_max_tokens),
            temperature=float(request.temperature), top_p=float(request.top_p), top_k=int(request.top_k),
            seed=request.seed, stop_token_ids=stop_token_ids(state.tokenizer),
            eos_token_id=first_eos_token_id(state.tokenizer))
        if len(prompt) + 1 > state.max_model_len:
            raise HTTPException(status_code=400, detail=f"prompt has {len(prompt)} tokens; the model context is "
                                                        f"{state.max_model_len}")
        item = PendingRequest(request=request, prompt=prompt, key=key,
                              future=asyncio.get_running_loop().create_future())
        if state.closing:
            raise HTTPException(status_code=503, detail="server is shutting down")
        task = asyncio.create_task(run_request_task(state, item))
        state.active_tasks.add(task)
        task.add_done_callback(state.active_tasks.discard)
        return await await_pending_response(state, raw_request, item)

    return app


@click.command(name="serve", context_settings={"help_option_names": ["-h", "--help"]})
@click.option("--model-path", required=True, help="Local checkpoint / tokenizer path or Hugging Face repo id.")
@click.option("--tp-size", type=int, default=1, show_default=True, help="Tensor parallel size.")
@click.option("--world-size", type=int, default=1, show_default=True, help="Total number of local worker ranks.")
@click.option("--host", default="0.0.0.0", show_default=True, help="HTTP bind host.")
@click.option("--port", type=int, default=8000, show_default=True, help="HTTP bind port.")
@click.option("--max-running-prompts", type=int, default=16, show_default=True,
              help="Upper bound of sequences decoded concurrently per data-parallel row.")
@click.option("--default-max-tokens", type=int, default=1024, show_default=True, help="Default max generated tokens.")
@click.option("--decode-progress-interval-s", type=float, default=0.0, show_default=True,
              help="Log decode progress every this many seconds (0 disables).")
@click.option("--eager-decode", is_flag=True, help="Run decode eagerly instead of replaying CUDA graphs.")
@click.option("--attn-backend", type=click.Choice(["flash", "native"]), default="flash", show_default=True)
@click.option("--kv-dtype", type=click.Choice(["bf16", "fp8"]), default="bf16", show_default=True)
@click.option("--disable-thinking", is_flag=True, help="Render chat templates with enable_thinking=False.")
def serve_command(model_path, tp_size, world_size, host, port, max_running_prompts, default_max_tokens,
                  decode_progress_interval_s, eager_decode, attn_backend, kv_dtype, disable_thinking) -> None:
    """Serve an OpenAI-compatible chat API."""
    import uvicorn

    from .model_refs import resolve_model_path

    if max_running_prompts < 1:
        raise click.UsageError("--max-running-prompts must be positive")
    if default_max_tokens < 1:
        raise click.UsageError("--default-max-tokens must be positive")
    app = create_app(model_path=resolve_model_path(model_path), tp_size=tp_size, world_size=world_size,
                     max_running_prompts=max_running_prompts, default_max_tokens=default_max_tokens,
                     decode_progress_interval_s=decode_progress_interval_s, eager_decode=eager_decode,
                     attn_backend=attn_backend, kv_dtype=kv_dtype,
                     chat_template_enable_thinking=False if disable_thinking else None)
    uvicorn.run(app, host=host, port=port)


def main() -> None:
    serve_command.main(prog_name="areno serve")


if __name__ == "__main__":
    main()
