"""Reference / critic / reward roles on a CPU rank worker: log-probs aligned with the input tokens, values per position,
rewards at the last token, scoring under a token budget in any row order, the clipped value loss against a hand-written
formula and its effect over a few steps, scalar heads found in checkpoints, and roles that cannot do what is asked."""

from __future__ import annotations

import json
import os

import pytest
import torch
from safetensors.torch import save_file

from areno_b200.api.backend.native import make_train_pack
from areno_b200.api.models import TrainSequence
from areno_b200.api.roles import ModelRole
from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig
from areno_b200.engine.roles import find_head_tensors
from areno_b200.engine.worker import RankWorker
from areno_b200.models.dense import TrainMeta
from areno_b200.ops.attention import build_varlen_meta
from areno_b200.parallel.context import single_process_context
from tests.helpers import tiny_config, write_tiny_checkpoint


@pytest.fixture()
def worker():
    single_process_context()
    cfg = EngineConfig(model=tiny_config(), model_path="", dummy_load=True, seed=3,
                       optimizer=OptimizerConfig(lr=1e-2, weight_decay=0.0, grad_clip_norm=1.0),
                       runtime=RuntimeConfig(eager_decode=True, max_model_len=128, activation_checkpointing=False))
    return RankWorker(cfg, "cpu")


def _rows(seed=0, lengths=(9, 1, 14, 5, 7)):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, 512, (n,), generator=g).tolist() for n in lengths]


def _manual_logprobs(model, row):
    ids = torch.tensor(row)
    with torch.no_grad():
        h = model(ids, torch.arange(len(row)), TrainMeta(build_varlen_meta([len(row)]), False)).hidden_states
        lp = torch.log_softmax(model.compute_logits(h).float(), -1)[:-1].gather(-1, ids[1:, None]).squeeze(-1)
    return [0.0] + lp.tolist()


def test_reference_scores_are_aligned_with_the_tokens_and_independent_of_batching(worker):
    roles = worker.role_manager()
    roles.ensure_roles({"actor": ModelRole("actor", "", True), "ref": ModelRole("ref", "", False)})
    assert set(roles.roles) == {"ref"}                      # the actor is the worker's own model, not a role copy
    assert not any(p.requires_grad for p in roles.roles["ref"].model.parameters())
    rows = _rows()
    ref = roles.score_logprobs("ref", rows)
    assert [len(r) for r in ref] == [len(r) for r in rows] and ref[1] == [0.0]
    for row, got in zip(rows, ref):
        assert got == pytest.approx(_manual_logprobs(worker.model, row), abs=1e-5)
    # one row per micro-batch, a tiny token budget, another order: the same numbers
    roles.score_token_budget = 10
    again = roles.score_logprobs("ref", list(reversed(rows)), microbatch_size=1)
    for a, b in zip(reversed(again), ref):
        assert a == pytest.approx(b, abs=1e-5)
    assert roles.score_logprobs("actor", rows[:1])[0] == pytest.approx(ref[0], abs=1e-5)
    assert roles.score_logprobs("ref", []) == []


def test_ensure_roles_is_idempotent_and_copies_share_nothing(worker):
    roles = worker.role_manager()
    spec = {"ref": ModelRole("ref", "", False)}
    roles.ensure_roles(spec)
    first = roles.roles["ref"]
    roles.ensure_roles(spec)
    assert roles.roles["ref"] is first
    a = next(worker.model.parameters())
    b = next(first.model.parameters())
    assert torch.equal(a, b) and a.data_ptr() != b.data_ptr()           # training the actor must not move the reference


def test_critic_values_and_the_clipped_value_loss(worker):
    roles = worker.role_manager()
    roles.ensure_roles({"critic": ModelRole("critic", "", True, optimizer_lr=5e-3)})
    critic = roles.roles["critic"]
    assert critic.optimizer is not None and critic.optimizer.lr == 5e-3 and float(critic.value_head.weight.detach().abs().sum()) == 0.0
    rows = _rows(1, (8, 6))
    values = roles.score_values("critic", rows)
    assert [len(v) for v in values] == [8, 6] and all(x == 0.0 for v in values for x in v)     # zero head: zero values
    assert roles.score_rewards("critic", rows) == [0.0, 0.0]

    def batch():
        seqs = []
        for row, n_p in zip(rows, (3, 2)):
            n = len(row)
            resp = [i >= n_p for i in range(n)]
            seqs.append(TrainSequence(tokens=row, prompt_mask=[not r for r in resp], logprobs=[0.0] * n, advantages=[0.0] * n,
                                      values=[0.0] * n, returns=[1.0 if r else 0.0 for r in resp]))
        return make_train_pack(seqs)

    stats = roles.train_values("critic", [batch()], cliprange_value=0.2, value_loss_coef=0.5)
    # zero predictions, zero old values, returns 1 on every response token: unclipped and clipped errors are both 1
    assert stats["critic_value_loss"] == pytest.approx(0.5 * 0.5 * 1.0) and stats["critic_value_mse"] == pytest.approx(1.0)
    assert stats["critic_value_target_mean"] == pytest.approx(1.0) and stats["critic_old_value_mean"] == 0.0
    assert stats["critic_value_clipfrac"] == 0.0
    losses = [stats["critic_value_loss"]]
    for _ in range(6):
        losses.append(roles.train_values("critic", [batch()], cliprange_value=10.0, value_loss_coef=0.5)["critic_value_loss"])
    assert losses[-1] < 0.5 * losses[0]                                  # the critic learns the constant return
    after = roles.score_values("critic", rows)
    assert sum(after[0][2:]) / len(after[0][2:]) > 0.2                   # predictions moved towards 1 where trained


def test_value_loss_takes_the_larger_of_the_clipped_and_unclipped_error(worker):
    roles = worker.role_manager()
    roles.ensure_roles({"critic": ModelRole("critic", "", True)})
    row = _rows(2, (6,))[0]
    seq = TrainSequence(tokens=row, prompt_mask=[True, True, False, False, False, False], logprobs=[0.0] * 6,
                        advantages=[0.0] * 6, values=[0, 0, 2.0, 2.0, -1.0, 0.5], returns=[0, 0, 3.0, 1.0, 0.0, 0.25])
    stats = roles.train_values("critic", [make_train_pack([seq])], cliprange_value=0.5, value_loss_coef=1.0)
    pred = torch.zeros(4)                                                # zero head
    old, target = torch.tensor([2.0, 2.0, -1.0, 0.5]), torch.tensor([3.0, 1.0, 0.0, 0.25])
    clipped = old + (pred - old).clamp(-0.5, 0.5)
    want = 0.5 * torch.maximum((pred - target) ** 2, (clipped - target) ** 2).mean()
    assert stats["critic_value_loss"] == pytest.approx(float(want), rel=1e-5)
    assert stats["critic_value_clipfrac"] == pytest.approx(float(((clipped - target) ** 2 > (pred - target) ** 2).float().mean()))


def test_roles_that_cannot_do_what_is_asked(worker, tmp_path):
    roles = worker.role_manager()
    roles.ensure_roles({"ref": ModelRole("ref", "", False)})
    with pytest.raises(RuntimeError, match="not a trainable value model"):
        roles.train_values("ref", [])
    with pytest.raises((RuntimeError, ValueError, KeyError)):
        roles.score_values("ref", _rows())
    ckpt = str(tmp_path / "no_head")
    write_tiny_checkpoint(ckpt)
    with pytest.raises(ValueError, match="has no scalar head"):
        roles.ensure_roles({"reward": ModelRole("reward", ckpt, False)})


def test_reward_models_bring_their_scalar_head(worker, tmp_path):
    ckpt = str(tmp_path / "rm")
    write_tiny_checkpoint(ckpt, seed=9)
    head = torch.full((1, 128), 0.01)
    save_file({"score.weight": head}, os.path.join(ckpt, "score_head.safetensors"))
    files = [f for f in os.listdir(ckpt) if f.endswith(".safetensors")]
    weight_map = {}
    from safetensors import safe_open

    for f in files:
        with safe_open(os.path.join(ckpt, f), framework="pt") as fh:
            weight_map.update({k: f for k in fh.keys()})
    json.dump({"metadata": {}, "weight_map": weight_map}, open(os.path.join(ckpt, "model.safetensors.index.json"), "w"))
    w, b = find_head_tensors(ckpt)
    assert torch.equal(w, head) and b is None and find_head_tensors(str(tmp_path)) == (None, None)
    roles = worker.role_manager()
    roles.ensure_roles({"reward": ModelRole("reward", ckpt, False)})
    rows = _rows(3, (7, 4))
    rewards = roles.score_rewards("reward", rows)
    per_token = roles.score_values("reward", rows)
    assert rewards == [pytest.approx(v[-1]) for v in per_token] and all(r != 0.0 for r in rewards)
    assert roles.roles["reward"].optimizer is None
