"""Agentic rollouts on CPU: the local OpenAI-compatible proxy, multi-turn trajectory accumulation
(prefix sharing, loss masks for tool results), reward records, and a training step on the batch."""

from __future__ import annotations

import asyncio
import json
import urllib.request

import pytest

from areno_b200.api import ArenoConfig, SamplingParams, Trainer, TrainSequence, grpo_loss_fn
from areno_b200.api.agentic import AgentBatch, AgentTrajectory, AgentTrajectoryTurn, LossMaskPolicy
from areno_b200.api.data import PromptBatch, PromptItem
from areno_b200.api.rewards import compute_group_advantages
from tests.helpers import FakeTokenizer, write_tiny_checkpoint


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("agentic") / "tiny")
    write_tiny_checkpoint(path, seed=3)
    return path


class ChatTokenizer(FakeTokenizer):
    """Round-trips generated ids (id t <-> word ``w<t>``) and renders chats as ``role: content`` lines."""

    chat_template = "role: content"

    def encode(self, text, add_special_tokens=True):
        out = []
        for w in str(text).split():
            if w.startswith("w") and w[1:].isdigit():
                out.append(int(w[1:]))
            else:
                out.extend(super().encode(w))
        return out or [3]

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(f"w{int(t)}" for t in ids)

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, **_kw):
        text = " ".join(f"{m['role']}: {m.get('content') or ''}" for m in messages)
        if add_generation_prompt:
            text += " assistant:"
        return self.encode(text) if tokenize else text


def _post(url: str, body: dict) -> tuple[int, dict]:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=60) as resp:
            return resp.status, json.loads(resp.read())
    except urllib.error.HTTPError as exc:
        return exc.code, json.loads(exc.read() or b"{}")


def test_proxy_multi_turn_trajectory_to_training_step(ckpt):
    cfg = ArenoConfig(tp_size=1, max_running_prompts=8, decode_progress_interval_s=0.0, launcher="inprocess",
                      optimizer={"lr": 1e-3}, runtime={"max_model_len": 256})
    trainer = Trainer(1, ckpt, custom_config=cfg)
    tok = ChatTokenizer()
    trainer.init(tokenizer=tok, eos_ids=(2,))
    params = SamplingParams(max_new_tokens=5, temperature=1.0, ignore_eos=True)
    items = [PromptItem(record={"prompt": "first question here", "answer": "42"}, prompt="first question here",
                        solutions=["42"], input_tokens=tok.encode("first question here")),
             PromptItem(record={"prompt": "second one", "answer": "7"}, prompt="second one", solutions=["7"],
                        input_tokens=tok.encode("second one"))]
    batch = AgentBatch.from_prompt_batch(PromptBatch(items=items, scanned=2, skipped_long=0, total_skipped_long=0),
                                         n_samples=2)
    assert len(batch) == 4

    async def play(session, item):
        url = session.get_base_url() + "/chat/completions"
        loop = asyncio.get_running_loop()
        messages = [{"role": "user", "content": item.prompt}]
        turns = []
        status, first = await loop.run_in_executor(None, _post, url, {"messages": messages, "model": "policy"})
        assert status == 200 and first["areno"]["response_tokens"] and first["choices"][0]["finish_reason"] == "stop"
        turns.append(AgentTrajectoryTurn(item=item, messages=list(messages), response=first))
        messages = messages + [{"role": "assistant", "content": first["choices"][0]["message"]["content"]},
                               {"role": "tool", "name": "lookup", "content": "tool says hello"}]
        status, second = await loop.run_in_executor(None, _post, url, {"messages": messages, "max_tokens": 3})
        assert status == 200 and len(second["areno"]["response_tokens"]) == 3
        turns.append(AgentTrajectoryTurn(item=item, messages=list(messages), response=second))
        return AgentTrajectory(turns=turns)

    async def scenario():
        async with trainer.rollout_session(sampling_params=params, loss_mask_policy=LossMaskPolicy(),
                                           max_running_prompts=4, timeout_s=60) as session:
            bad, _ = await asyncio.get_running_loop().run_in_executor(
                None, _post, session.get_base_url() + "/chat/completions", {"messages": []})
            assert bad == 400
            trajs = await asyncio.gather(*[play(session, it) for it in batch.iter_samples()])
            samples = session.accumulate(list(trajs))
            return session.build_train_batch(samples, lambda rec: float(len(rec.tool_results) == 1 and rec.answer in ("42", "7")))

    tb = asyncio.run(scenario())
    try:
        assert len(tb.token_rows) == 4 and tb.rewards == [1.0] * 4
        for row, resp_mask, loss_mask, lps in zip(tb.token_rows, tb.response_masks, tb.loss_masks, tb.rollout_logprobs):
            assert len(row) == len(resp_mask) == len(loss_mask) == len(lps)
            # two assistant spans (5 + 3 generated tokens) are trained on; the tool result between them is
            # context only (part of the row, neither response nor loss)
            assert sum(loss_mask) == 8 and sum(resp_mask) == 8
            first = resp_mask.index(True)
            spans = "".join("1" if m else "0" for m in resp_mask[first:])
            assert spans.startswith("11111") and spans.endswith("111") and "0" in spans
            tool_ids = tok.encode("tool says hello")
            assert any(row[i:i + len(tool_ids)] == tool_ids for i in range(first + 5, len(row) - 3))
        assert tb.reward_records[0].tool_results[0]["content"] == "tool says hello"
        seqs = []
        for g in range(2):
            adv = compute_group_advantages([1.0, 0.0])
            for j in range(2):
                i = g * 2 + j
                row = tb.token_rows[i]
                seqs.append(TrainSequence(tokens=row, prompt_mask=[not m for m in tb.response_masks[i]],
                                          loss_mask=tb.loss_masks[i], logprobs=tb.rollout_logprobs[i],
                                          advantages=[adv[j]] * len(row), reward=tb.rewards[i], eos_token_id=2))
        stats = trainer.train(seqs, grpo_loss_fn, mini_bs=2)
        assert stats["num_microbatches"] == 2 and stats["grad_norm"] > 0
    finally:
        trainer.close()
