"""PPO batch assembly on the CPU with scripted role scores: where old log-probs, values, returns and advantages land in
a row, the reward on the last response token, rows whose response is split by tool results, rows without loss tokens,
advantage standardisation, critic warm-up and the reward model as a role."""

from __future__ import annotations

import logging
from types import SimpleNamespace

import pytest

from areno_b200.api.models import TrainSequence
from areno_b200.api.roles import MissingRoleCapability
from areno_b200.api.trainers.ppo import PPOTrainer, normalize_response_advantages, summary_stats


class Roles:
    """Scores that encode the position: old log-prob of token i is -(i), reference -(i) - 0.5, value before i+1 is i."""

    def __init__(self):
        self.calls = []

    def score_logprobs(self, role, rows):
        self.calls.append((role, "logprobs"))
        off = 0.5 if role == "ref" else 0.0
        return [[-(float(i)) - off for i in range(len(r))] for r in rows]

    def score_values(self, role, rows):
        self.calls.append((role, "values"))
        return [[float(i) for i in range(len(r))] for r in rows]

    def score_rewards(self, role, rows):
        self.calls.append((role, "rewards"))
        return [float(len(r)) for r in rows]

    def train_values(self, role, batch, mini_bs, accumulation, cliprange_value, value_loss_coef):
        self.calls.append((role, "train_values", len(batch), mini_bs, cliprange_value, value_loss_coef))
        return {"critic_value_loss": 0.25, "note": "text"}


def _trainer(reward_role=False, **cfg):
    t = object.__new__(PPOTrainer)
    base = dict(gamma=1.0, lam=1.0, mini_bs=4, gradient_accumulation_steps=None, value_clip_eps=0.3, value_loss_coef=0.7,
                critic_warmup_steps=2)
    base.update(cfg)
    t.config = SimpleNamespace(**base)
    t.areno = Roles()
    t.logger = logging.getLogger("test.ppo")
    t._last_ppo_stats = {}
    t.roles = {"actor": 1, "ref": 2, "critic": 3}
    if reward_role:
        t.roles["reward"] = 4
    return t


TOK = SimpleNamespace(eos_token_id=2)


def test_single_span_rows_place_signals_on_the_response_tokens():
    t = _trainer()
    rows = [[10, 11, 12, 13, 14]]
    rmask = [[False, False, True, True, True]]
    batch, rewards, rollout_lp = t._build_ppo_batch(TOK, rows, rmask, [list(rmask[0])], [[0, 0, -0.1, -0.2, -0.3]], [2.0],
                                                    explicit_loss_mask=False)
    seq = batch[0]
    assert rewards == [2.0] and rollout_lp == [-0.1, -0.2, -0.3] and seq.reward == 2.0 and seq.eos_token_id == 2
    assert seq.prompt_mask == [True, True, False, False, False] and seq.loss_mask == []
    assert seq.logprobs == [0.0, 0.0, -2.0, -3.0, -4.0]                       # the actor's re-scored values, by position
    assert seq.values == [0.0, 0.0, 1.0, 2.0, 3.0]                            # V before token i sits at i - 1 in the row
    # gamma = lam = 1: every action's return is the final reward, its advantage reward - V
    assert seq.returns == [0.0, 0.0, 2.0, 2.0, 2.0]
    raw = [2.0 - 1.0, 2.0 - 2.0, 2.0 - 3.0]
    mean, std = 0.0, (2 / 3) ** 0.5
    assert seq.advantages[2:] == pytest.approx([(a - mean) / std for a in raw]) and seq.advantages[:2] == [0.0, 0.0]
    assert seq.ref_logprobs == [-0.5, -1.5, -2.5, -3.5, -4.5]
    stats = t._last_ppo_stats
    assert stats["critic_value_loss"] == 0.25 and "note" not in stats
    assert stats["old_rollout_logprob_diff_mean"] == pytest.approx((-1.9 - 2.8 - 3.7) / 3)
    assert stats["return_mean"] == 2.0 and stats["gae_advantage_mean"] == pytest.approx(0.0)
    assert stats["normalized_advantage_std"] == pytest.approx(1.0)
    assert ("critic", "train_values", 1, 4, 0.3, 0.7) in t.areno.calls
    assert [c[:2] for c in t.areno.calls[:3]] == [("ref", "logprobs"), ("actor", "logprobs"), ("critic", "values")]


def test_rows_split_by_tool_results_gather_every_signal_by_position():
    t = _trainer()
    #        prompt   span 1    tool result   span 2
    rmask = [False, False, True, True, False, False, True, True]
    lmask = list(rmask)
    rows = [list(range(20, 28))]
    roll = [0, 0, -0.1, -0.2, 0, 0, -0.3, -0.4]
    batch, _, rollout_lp = t._build_ppo_batch(TOK, rows, [rmask], [lmask], [roll], [1.0], explicit_loss_mask=True)
    seq = batch[0]
    assert rollout_lp == [-0.1, -0.2, -0.3, -0.4]
    assert seq.logprobs == [0, 0, -2.0, -3.0, 0, 0, -6.0, -7.0]               # not -4, -5: those are tool-result tokens
    assert seq.values == [0, 0, 1.0, 2.0, 0, 0, 5.0, 6.0]
    assert seq.returns == [0, 0, 1.0, 1.0, 0, 0, 1.0, 1.0]
    assert seq.loss_mask == lmask and seq.prompt_mask == [not r for r in rmask]
    assert seq.advantages[4] == seq.advantages[5] == 0.0 and seq.advantages[2] > seq.advantages[7]
    assert t._last_ppo_stats["old_logprob_min"] == -7.0 and t._last_ppo_stats["critic_value_max"] == 6.0


def test_masked_response_tokens_keep_returns_but_get_no_advantage():
    t = _trainer()
    rmask = [False, True, True, True]
    lmask = [False, True, False, True]
    batch, _, rollout_lp = t._build_ppo_batch(TOK, [[1, 2, 3, 4]], [rmask], [lmask], [[0, -1.0, -2.0, -3.0]], [3.0],
                                              explicit_loss_mask=True)
    seq = batch[0]
    assert rollout_lp == [-1.0, -3.0] and seq.advantages[2] == 0.0 and seq.returns[2] == 3.0 and seq.values[2] == 1.0
    assert seq.advantages[1] == pytest.approx(1.0) and seq.advantages[3] == pytest.approx(-1.0)   # standardised over 2


def test_rows_without_response_or_loss_tokens_are_left_out():
    t = _trainer()
    rows = [[1, 2, 3], [4, 5, 6], [7, 8, 9]]
    rmasks = [[False, False, False], [False, True, True], [False, True, True]]
    lmasks = [[False, False, False], [False, False, False], [False, True, True]]
    batch, rewards, _ = t._build_ppo_batch(TOK, rows, rmasks, lmasks, [[0, 0, 0]] * 3, [1.0, 2.0, 3.0], explicit_loss_mask=True)
    assert len(batch) == 1 and batch[0].tokens == [7, 8, 9] and rewards == [1.0, 2.0, 3.0]
    t2 = _trainer()
    batch, _, _ = t2._build_ppo_batch(TOK, rows[:1], rmasks[:1], lmasks[:1], [[0, 0, 0]], [1.0], explicit_loss_mask=True)
    assert batch == [] and not any(c[1] == "train_values" for c in t2.areno.calls)


def test_misaligned_rows_and_scores_are_errors():
    t = _trainer()
    with pytest.raises(ValueError, match="misaligned token/mask"):
        t._build_ppo_batch(TOK, [[1, 2, 3]], [[False, True]], [[False, True, True]], [[0, 0, 0]], [1.0], explicit_loss_mask=True)
    t.areno.score_values = lambda role, rows: [[0.0] for _ in rows]
    with pytest.raises(ValueError, match="misaligned token values"):
        t._build_ppo_batch(TOK, [[1, 2, 3]], [[False, True, True]], [[False, True, True]], [[0, 0, 0]], [1.0],
                           explicit_loss_mask=True)
    t = _trainer()
    t.areno.score_logprobs = lambda role, rows: [[0.0] for _ in rows]
    with pytest.raises(ValueError, match="misaligned old logprobs"):
        t._build_ppo_batch(TOK, [[1, 2, 3]], [[False, True, True]], [[False, True, True]], [[0, 0, 0]], [1.0],
                           explicit_loss_mask=True)


def test_discounting_follows_the_response_tokens():
    t = _trainer(gamma=0.5, lam=0.0)
    batch, _, _ = t._build_ppo_batch(TOK, [[1, 2, 3]], [[False, True, True]], [[False, True, True]], [[0, 0, 0]], [4.0],
                                     explicit_loss_mask=False)
    # lam 0: one-step errors; V = [0, 1] before the two actions: delta0 = 0 + 0.5 * 1 - 0, delta1 = 4 - 1
    assert batch[0].returns[1:] == pytest.approx([0.5 + 0.0, 3.0 + 1.0])


def test_the_reward_model_scores_when_there_is_no_reward_function():
    t = _trainer(reward_role=True)
    batch, rewards, _ = t._build_ppo_batch(TOK, [[1, 2, 3], [4, 5, 6, 7]], [[False, True, True], [False, False, True, True]],
                                           [[False, True, True], [False, False, True, True]], [[0] * 3, [0] * 4], None,
                                           explicit_loss_mask=False)
    assert rewards == [3.0, 4.0] and t.areno.calls[0] == ("reward", "rewards")
    assert t._last_ppo_stats["reward_model_raw_reward_max"] == 4.0 and "reward_score_time_s" in t._last_ppo_stats
    with pytest.raises(MissingRoleCapability, match="reward"):
        _trainer()._build_ppo_batch(TOK, [[1, 2]], [[False, True]], [[False, True]], [[0, 0]], None, explicit_loss_mask=False)


def test_prompt_rollouts_and_agentic_batches_share_the_assembly():
    t = _trainer()
    t.reward_fn = lambda rec: float(len(rec.completion.split()))
    tok = SimpleNamespace(eos_token_id=2, decode=lambda ids: " ".join(str(i) for i in ids))
    item = SimpleNamespace(input_tokens=[5, 6], prompt="p", record={"id": 1}, solutions=["s"])
    result = SimpleNamespace(sequences=[SimpleNamespace(resp_tokens=[7, 8, 9], resp_logprobs=[-0.1, -0.2, -0.3]),
                                        SimpleNamespace(resp_tokens=[7], resp_logprobs=[-0.4])])
    batch, rewards, rollout_lp = t._materialize_train_batch(tok, SimpleNamespace(items=[item]), [result])
    assert rewards == [3.0, 1.0] and rollout_lp == [-0.1, -0.2, -0.3, -0.4] and [len(s.tokens) for s in batch] == [5, 3]
    assert batch[0].loss_mask == [] and "reward_score_time_s" in t._last_ppo_stats
    agent = SimpleNamespace(token_rows=[[5, 6, 7]], response_masks=[[False, True, True]], loss_masks=[[False, True, False]],
                            rollout_logprobs=[[0, -0.5, -0.6]], rewards=[1])
    batch, rewards, rollout_lp = t._materialize_agentic_train_batch(tok, None, agent)
    assert rewards == [1.0] and rollout_lp == [-0.5] and batch[0].loss_mask == [False, True, False]


def test_advantages_are_standardised_over_loss_tokens_only():
    a = TrainSequence(tokens=[1, 2, 3], prompt_mask=[True, False, False], advantages=[9.0, 1.0, 3.0])
    b = TrainSequence(tokens=[1, 2, 3], prompt_mask=[True, False, False], loss_mask=[False, False, True], advantages=[9.0, 9.0, 5.0])
    normalize_response_advantages([a, b])
    vals = [1.0, 3.0, 5.0]
    std = (sum((v - 3.0) ** 2 for v in vals) / 3) ** 0.5
    assert a.advantages == pytest.approx([0.0, -2.0 / std, 0.0]) and b.advantages == pytest.approx([0.0, 0.0, 2.0 / std])
    c = TrainSequence(tokens=[1, 2], prompt_mask=[True, False], advantages=[0.0, 4.0])
    normalize_response_advantages([c])
    assert c.advantages == [0.0, 0.0]                                   # one value: centred, not divided by zero
    normalize_response_advantages([TrainSequence(tokens=[1], prompt_mask=[True], advantages=[1.0])])
    assert summary_stats("x", []) == {} and summary_stats("x", [1.0, 3.0]) == {"x_mean": 2.0, "x_std": 1.0, "x_min": 1.0,
                                                                               "x_max": 3.0}


def test_the_actor_waits_for_the_critic_warm_up_and_results_carry_the_ppo_statistics():
    t = _trainer(critic_warmup_steps=2)
    assert [t._should_train_policy(s) for s in range(4)] == [False, False, True, True]
    assert t._policy_role_name() == "actor"
    t._last_ppo_stats = {"critic_value_loss": 0.1}
    assert t._augment_train_stats({"loss": 1.0}) == {"loss": 1.0, "critic_value_loss": 0.1}
    assert t._augment_train_stats(None) is None
