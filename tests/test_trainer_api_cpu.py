"""``Trainer`` bookkeeping against a fake backend: step accounting, nested rollout sessions, timings attached to the
train result, prompt batching with over-long prompts skipped, role calls passed through, metrics recorded."""

from __future__ import annotations

import asyncio
import json

import pytest

from areno_b200.api import SamplingParams, Trainer, TrainSequence
from areno_b200.api.context import Context

from .helpers import FakeTokenizer


class FakeBackend:
    def __init__(self):
        self.calls = []

    def close(self):
        self.calls.append("close")

    def begin_rollout_session(self, ctx):
        self.calls.append(("begin", ctx.global_step))

    async def begin_rollout_session_async(self, ctx):
        self.calls.append(("begin_async", ctx.global_step))

    def end_rollout_session(self, ctx):
        self.calls.append(("end", ctx.global_step))

    async def end_rollout_session_async(self, ctx):
        self.calls.append(("end_async", ctx.global_step))

    async def sync_rollout_session_async(self, ctx):
        self.calls.append(("sync", ctx.global_step))

    def rollout_batch(self, ctx, prompt_tokens, n_samples, params):
        self.calls.append(("rollout", ctx.global_step, [list(p) for p in prompt_tokens], n_samples))
        return [f"result{i}" for i in range(len(prompt_tokens))]

    async def rollout_batch_async(self, ctx, prompt_tokens, n_samples, params):
        return self.rollout_batch(ctx, prompt_tokens, n_samples, params)

    def train(self, ctx, batch, loss_fn, mini_bs, accum):
        self.calls.append(("train", ctx.global_step, len(batch), mini_bs, accum))
        return {"loss": 0.5, "grad_norm": 1.0}

    def dp_size(self, ctx):
        return 4

    def ensure_roles(self, ctx, roles):
        self.calls.append(("roles", sorted(roles)))

    def score_logprobs(self, ctx, role, rows, microbatch_size=8):
        return [[-1.0] * len(r) for r in rows] + [microbatch_size]

    def score_values(self, ctx, role, rows):
        return [[0.0] * len(r) for r in rows]

    def score_rewards(self, ctx, role, rows):
        return [float(len(r)) for r in rows]

    def train_values(self, ctx, role, batch, mini_bs, accum, *, cliprange_value, value_loss_coef):
        return {"value_loss": cliprange_value * value_loss_coef}

    def save_checkpoint(self, ctx, path):
        return path


def _trainer(metrics_dir=None):
    t = Trainer(1, "unused-path", metrics_log_dir=metrics_dir, score_micro_bs=3)
    t._tokenizer = FakeTokenizer()
    t._backend = FakeBackend()
    t._ctx = Context(1, "unused-path", t._tokenizer)
    t._initialized = True
    return t


def _seq():
    return TrainSequence(prompt_mask=[True, False], tokens=[5, 6], logprobs=[0.0, -0.1], advantages=[0.0, 1.0], reward=1.0,
                         eos_token_id=2)


def test_uninitialised_trainer_refuses_work():
    t = Trainer(1, "unused-path")
    assert t.global_step == -1
    with pytest.raises(RuntimeError):
        t.train([_seq()], lambda pack, lp: lp.sum())
    with pytest.raises(RuntimeError):
        t.begin_rollout_session()
    t.close()                                   # closing twice or before init is harmless
    t.close()


def test_one_step_spans_session_rollouts_and_train():
    t = _trainer()
    params = SamplingParams(max_new_tokens=4)
    with pytest.raises(RuntimeError):
        t.rollout_token_batch([[1, 2]], 2, params)                 # only inside a session
    with pytest.raises(TypeError):
        t.train([_seq()], "not callable")
    t.begin_rollout_session()
    t.begin_rollout_session()                                      # nested: the backend sees one session
    assert t.rollout_token_batch([[1, 2], [3]], 2, params) == ["result0", "result1"]
    t.end_rollout_session()
    assert ("end", 0) not in t._backend.calls                      # still open: depth 1
    t.end_rollout_session()
    t.end_rollout_session()                                        # extra end is ignored
    out = t.train([_seq(), _seq()], lambda pack, lp: lp.sum(), mini_bs=2, gradient_accumulation_steps=1)
    assert t.global_step == 0                                      # session + rollouts + train = step 0
    assert out["loss"] == 0.5 and out["step_rollout_time_s"] >= 0 and out["step_train_time_s"] >= 0 and out["step_e2e_time_s"] >= 0
    kinds = [c[0] if isinstance(c, tuple) else c for c in t._backend.calls]
    assert kinds == ["begin", "rollout", "end", "train"]
    assert t._backend.calls[1] == ("rollout", 0, [[1, 2], [3]], 2) and t._backend.calls[3] == ("train", 0, 2, 2, 1)
    # the next train call alone is the next step, and carries no stale rollout time
    out2 = t.train([_seq()], lambda pack, lp: lp.sum())
    assert t.global_step == 1 and "step_rollout_time_s" not in out2
    t.close()
    assert t._backend is None


def test_async_sessions_and_sync_guard():
    t = _trainer()

    async def run():
        with pytest.raises(RuntimeError):
            await t.sync_rollout_session_async()
        await t.begin_rollout_session_async()
        await t.sync_rollout_session_async()
        res = await t.rollout_token_batch_async([[7, 8, 9]], 1, SamplingParams(max_new_tokens=2))
        await t.end_rollout_session_async()
        return res

    assert asyncio.run(run()) == ["result0"]
    assert [c[0] for c in t._backend.calls] == ["begin_async", "sync", "rollout", "end_async"]


def test_prompt_batches_skip_long_prompts_and_keep_records():
    t = _trainer()
    data = [{"prompt": "one two", "answer": "a"}, {"prompt": "w " * 40, "answer": "b"}, {"prompt": "three", "answer": "c"},
            {"prompt": "four five six", "answer": "d"}]
    batches = list(t.load_prompt_batches(data, batch_size=2, max_prompt_tokens=8))
    assert [len(b.items) for b in batches] == [2, 1]
    assert batches[0].scanned == 3 and batches[0].skipped_long == 1 and batches[1].total_skipped_long == 1
    assert [i.record["answer"] for b in batches for i in b.items] == ["a", "c", "d"]
    assert batches[0].items[0].input_tokens == t.get_tokenizer().encode("one two")
    with pytest.raises(ValueError):
        list(t.load_prompt_batches([{"question": "q"}], batch_size=1, max_prompt_tokens=8))


def test_role_calls_pass_through_with_the_configured_micro_batch():
    t = _trainer()
    t.ensure_roles({"ref": object(), "critic": object()})
    assert t._backend.calls[-1] == ("roles", ["critic", "ref"])
    assert t.score_logprobs("ref", [[1, 2, 3]]) == [[-1.0, -1.0, -1.0], 3]          # score_micro_bs reaches the backend
    assert t.score_values("critic", [[1, 2]]) == [[0.0, 0.0]] and t.score_rewards("reward", [[1, 2, 3, 4]]) == [4.0]
    assert t.train_values("critic", [_seq()], 4, cliprange_value=0.2, value_loss_coef=0.5) == {"value_loss": 0.1}
    assert t.dp_size() == 4


def test_metrics_are_recorded_per_train_call(tmp_path, monkeypatch):
    from areno_b200.api import metrics

    monkeypatch.setattr(metrics, "create_tensorboard_writer", lambda d: metrics.JsonlScalarWriter(d))
    t = _trainer(str(tmp_path))
    t.begin_rollout_session()
    t.end_rollout_session()
    t.train([_seq(), _seq()], lambda pack, lp: lp.sum())
    t.close()
    rows = [json.loads(line) for line in open(tmp_path / "metrics.jsonl")]
    tags = {r["tag"] for r in rows}
    assert {"rollout/rewards_mean", "rollout/num_sequences", "train/loss", "time/train", "time/rollout"} <= tags
    assert all(r["step"] == 0 for r in rows)


def test_phase_timers_show_up_in_the_train_result():
    from areno_b200.utils import tracing

    t = _trainer()
    tracing.configure(timers=True)
    try:
        tracing.phase_report()
        with tracing.trace_range("train/forward"):
            pass
        out = t.train([_seq()], lambda pack, lp: lp.sum())
    finally:
        tracing.configure(nvtx=False, timers=False)
    assert "device_ms/train/forward" in out
    assert not any(k.startswith("device_ms/") for k in t.train([_seq()], lambda pack, lp: lp.sum()))


def test_trainer_as_a_context_manager_closes_the_backend():
    t = _trainer()
    backend = t._backend
    with t as entered:
        assert entered is t and t._initialized
        t.train([_seq()], lambda pack, lp: lp.sum())
    assert backend.calls[-1] == "close" and t._backend is None
    with pytest.raises(RuntimeError):
        t.train([_seq()], lambda pack, lp: lp.sum())
