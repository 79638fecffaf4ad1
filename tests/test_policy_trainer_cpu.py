"""The policy trainer's loop on the CPU with a scripted SDK object: group advantages broadcast over response tokens,
agentic batches grouped by prompt, the step loop (rollout, train, save cadence, stop conditions, the skip path used
during critic warm-up), and completion logging."""

from __future__ import annotations

import logging
from contextlib import asynccontextmanager
from types import SimpleNamespace

import pytest

from areno_b200.api.data import PromptBatch, PromptItem
from areno_b200.api.models import RolloutResult, RolloutSequence
from areno_b200.api.rewards import RewardRecord
from areno_b200.api.trainers.base import BaseTrainer
from areno_b200.api.trainers.policy_only import PolicyOnlyTrainer


class Tok:
    eos_token_id = 2

    def decode(self, ids):
        return " ".join(str(i) for i in ids)


class ScriptedSdk:
    """What the trainer calls on ``Trainer``: prompt batches, a rollout session, train, save, step accounting."""

    def __init__(self, n_batches=3):
        self.n_batches, self.log, self.closed = n_batches, [], False

    def init(self):
        self.log.append("init")

    def close(self):
        self.closed = True

    def get_tokenizer(self):
        return Tok()

    def load_prompt_batches(self, dataset, batch_size, max_prompt_tokens):
        for b in range(self.n_batches):
            items = [PromptItem(prompt=f"p{b}{i}", solutions=[str(i)], input_tokens=[5, 6 + i], record={"k": i})
                     for i in range(batch_size)]
            yield PromptBatch(items=items, scanned=batch_size, skipped_long=0, total_skipped_long=0)

    @asynccontextmanager
    async def rollout_session(self, **kw):
        self.log.append(("session", kw.get("proxy"), kw.get("max_running_prompts")))
        yield self

    async def rollout_token_batch_async(self, tokens, n_samples, params):
        self.log.append(("rollout", len(tokens), n_samples, params.max_new_tokens))
        return [RolloutResult(sequences=[RolloutSequence(resp_tokens=[9] * (s + 1), resp_logprobs=[-0.5] * (s + 1))
                                         for s in range(n_samples)]) for _ in tokens]

    def train(self, batch, loss_fn, mini_bs, gradient_accumulation_steps):
        self.log.append(("train", len(batch), mini_bs))
        return {"loss": 0.5}

    def finish_step(self):
        self.log.append("finish_step")

    def save_checkpoint(self, path):
        self.log.append(("save", path))


def _trainer(sdk=None, **cfg):
    base = dict(epochs=1, batch_size=2, n_samples=2, max_prompt_tokens=16, max_new_tokens=4, max_context_len=None,
                greedy=False, temperature=1.0, top_k=-1, top_p=1.0, mini_bs=2, gradient_accumulation_steps=None,
                max_steps=None, save_path=None, save_interval=100, agent_fn=None, chat_template_enable_thinking=None,
                resolved_max_running_prompts=lambda: 8)
    base.update(cfg)
    sdk = sdk or ScriptedSdk()
    t = PolicyOnlyTrainer(SimpleNamespace(**base), instance=sdk, dataset=[], loss_fn=lambda *a: None,
                          reward_fn=lambda rec: float(len(rec.tokens) % 2))
    return t, sdk


def test_group_advantages_are_broadcast_over_the_response_tokens():
    t, _ = _trainer()
    item = PromptItem(prompt="p", solutions=["s"], input_tokens=[5, 6, 7], record={"id": 1})
    seen = []

    def reward(rec):
        seen.append(rec)
        return {1: 1.0, 2: 0.0, 3: 0.0}[len(rec.tokens) - 3]

    t.reward_fn = reward
    result = RolloutResult(sequences=[RolloutSequence(resp_tokens=[9] * n, resp_logprobs=[-0.1 * n] * n) for n in (1, 2, 3)])
    batch, rewards, rollout_lp = t._materialize_train_batch(Tok(), SimpleNamespace(items=[item]), [result])
    assert rewards == [1.0, 0.0, 0.0] and len(rollout_lp) == 6
    assert [s.prompt_mask for s in batch] == [[True] * 3 + [False] * n for n in (1, 2, 3)]
    assert batch[0].advantages[:3] == [0.0] * 3 and batch[0].advantages[3] > 0 > batch[1].advantages[3]
    assert batch[2].advantages[3:] == [batch[2].advantages[3]] * 3 and batch[1].logprobs == [0, 0, 0, -0.2, -0.2]
    assert batch[0].reward == 1.0 and batch[0].eos_token_id == 2
    rec = seen[1]
    assert rec.completion == "9 9" and rec.answer == ["s"] and rec.source_record == {"id": 1}
    assert rec.loss_mask == [False] * 3 + [True] * 2 and rec.metadata == {"prompt_index": 0, "sample_index": 1}


def test_agentic_rows_are_grouped_by_prompt_and_masked_tokens_carry_no_advantage():
    t, _ = _trainer()

    def rec(pi, si):
        return RewardRecord(prompt="p", completion="c", metadata={"prompt_index": pi, "sample_index": si})

    agent = SimpleNamespace(
        token_rows=[[1, 2, 3, 4], [1, 2, 5], [7, 8, 9]],
        response_masks=[[False, True, True, True], [False, True, True], [False, True, True]],
        loss_masks=[[False, True, False, True], [False, True, True], [False, True, True]],
        rollout_logprobs=[[0, -1.0, -2.0, -3.0], [0, -0.5, -0.5], [0, -0.1, -0.1]],
        rewards=[1, 0, 5], reward_records=[rec(0, 0), rec(0, 1), rec(1, 0)])
    batch, rewards, rollout_lp = t._materialize_agentic_train_batch(Tok(), None, agent)
    assert rewards == [1.0, 0.0, 5.0] and rollout_lp == [-1.0, -3.0, -0.5, -0.5, -0.1, -0.1]
    a0, a1, a2 = batch
    assert a0.advantages[1] == a0.advantages[3] > 0 and a0.advantages[2] == 0.0 and a0.advantages[0] == 0.0
    assert a1.advantages[1] == pytest.approx(-a0.advantages[1])            # normalised within prompt 0's two samples
    assert a2.advantages == [0.0, 0.0, 0.0]                                   # a group of one has no signal
    assert a0.loss_mask == [False, True, False, True] and a0.prompt_mask == [True, False, False, False]
    agent.rewards = None
    with pytest.raises(ValueError, match="requires a reward_fn"):
        t._materialize_agentic_train_batch(Tok(), None, agent)
    agent.rewards = [1, 0, 5]
    agent.loss_masks[0] = [False, True]
    with pytest.raises(ValueError, match="misaligned"):
        t._materialize_agentic_train_batch(Tok(), None, agent)


def test_the_loop_rolls_out_trains_saves_and_closes(tmp_path):
    t, sdk = _trainer(save_path=str(tmp_path), save_interval=2, epochs=1)
    t.fit()
    kinds = [e if isinstance(e, str) else e[0] for e in sdk.log]
    assert kinds == ["init"] + ["session", "rollout", "train"] * 2 + ["save"] + ["session", "rollout", "train"]
    assert sdk.log[1] == ("session", False, 8) and sdk.log[2] == ("rollout", 2, 2, 4) and sdk.log[3] == ("train", 4, 2)
    assert sdk.log[7] == ("save", str(tmp_path / "step_000002")) and sdk.closed


def test_max_steps_ends_the_run_across_epochs():
    t, sdk = _trainer(epochs=3, max_steps=4)
    t.fit()
    assert sum(1 for e in sdk.log if isinstance(e, tuple) and e[0] == "train") == 4 and sdk.closed


def test_a_failing_step_still_closes_the_backend():
    t, sdk = _trainer()
    sdk.train = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("device lost"))
    with pytest.raises(RuntimeError, match="device lost"):
        t.fit()
    assert sdk.closed


def test_skipped_policy_updates_close_the_step_and_do_not_save(tmp_path):
    t, sdk = _trainer(save_path=str(tmp_path), save_interval=1)
    t._should_train_policy = lambda step: step >= 2
    t._augment_train_stats = lambda r: dict(r, critic=1.0)
    t.fit()
    kinds = [e if isinstance(e, str) else e[0] for e in sdk.log]
    assert kinds.count("finish_step") == 2 and kinds.count("train") == 1 and kinds.count("save") == 1
    assert sdk.log[-1] == ("save", str(tmp_path / "step_000003"))


def test_save_cadence_and_stop_rule():
    t = object.__new__(BaseTrainer)
    t.logger = logging.getLogger("test.base")
    saved = []
    t.areno = SimpleNamespace(save_checkpoint=saved.append)
    t.config = SimpleNamespace(save_path="/out", save_interval=3, max_steps=5)
    for step in range(7):
        t._maybe_save(0, step)
    assert saved == ["/out/step_000003", "/out/step_000006"]
    assert [t._reached_max_steps(0, s) for s in (4, 5, 6)] == [False, True, True]
    t.config = SimpleNamespace(save_path=None, save_interval=1, max_steps=None)
    t._maybe_save(0, 0)
    assert len(saved) == 2 and not t._reached_max_steps(0, 10 ** 6)
    t.config = SimpleNamespace(save_path="/out", save_interval=0, max_steps=None)
    t._maybe_save(0, 0)
    assert len(saved) == 2


def test_completions_are_logged_only_on_request(monkeypatch, caplog):
    t, _ = _trainer()
    item = PromptItem(prompt="the prompt", solutions=None, input_tokens=[5, 6], record={})
    results = [RolloutResult(sequences=[RolloutSequence(resp_tokens=[9, 9], resp_logprobs=[0, 0])] * 3)]
    with caplog.at_level(logging.INFO):
        t._log_completions(Tok(), 0, 0, SimpleNamespace(items=[item]), results)
    assert "completion=" not in caplog.text
    monkeypatch.setenv("ARENO_LOG_COMPLETIONS", "2")
    with caplog.at_level(logging.INFO):
        t._log_completions(Tok(), 0, 0, SimpleNamespace(items=[item]), results)
    assert caplog.text.count("completion='9 9'") == 2 and "prompt='the prompt'" in caplog.text


def test_sampling_parameters_come_from_the_config():
    t, _ = _trainer(greedy=True, temperature=0.3, top_k=7, top_p=0.8, max_new_tokens=11, max_prompt_tokens=13, max_context_len=99)
    p = t._sampling_params()
    assert (p.greedy, p.temperature, p.top_k, p.top_p, p.max_new_tokens, p.max_prompt_len, p.max_context_len) == \
        (True, 0.3, 7, 0.8, 11, 13, 99)
    assert t._policy_role_name() == "policy" and t._should_train_policy(0) and not t._agentic_enabled()
