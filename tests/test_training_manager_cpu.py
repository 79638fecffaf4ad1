"""The training manager on the CPU: per-action log-probs of a packed batch equal those of every sequence run on its own;
micro-batches accumulate into one optimizer step whose update equals the update from the summed gradients; statistics
of a step; the loss function travels with the pack or comes from the manager."""

from __future__ import annotations

import pytest
import torch

from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig
from areno_b200.engine.training import TrainingManager, pack_train_data
from areno_b200.models.dense import DenseCausalLM, TrainMeta, init_weights
from areno_b200.ops.attention import build_varlen_meta
from areno_b200.parallel.context import single_process_context
from tests.helpers import tiny_config


def _manager(loss_fn=None, **ocfg):
    single_process_context()
    cfg = tiny_config(num_hidden_layers=2)
    model = DenseCausalLM(cfg)
    init_weights(model, 5)
    base = dict(lr=1e-2, weight_decay=0.0, grad_clip_norm=None)
    base.update(ocfg)
    econf = EngineConfig(model=cfg, optimizer=OptimizerConfig(**base), runtime=RuntimeConfig(activation_checkpointing=False))
    return TrainingManager(model, econf, "cpu", loss_fn=loss_fn), model


def _pack(lengths, seed=0, prompt=2):
    g = torch.Generator().manual_seed(seed)
    width = max(lengths)
    ids = torch.randint(3, 512, (len(lengths), width), generator=g)
    pm = torch.ones(len(lengths), width, dtype=torch.bool)
    for r, n in enumerate(lengths):
        pm[r, prompt:n] = False
    return {"input_ids": ids, "lengths": torch.tensor(lengths), "prompt_mask": pm,
            "logprobs": -torch.rand(len(lengths), width, generator=g), "advantages": torch.randn(len(lengths), width, generator=g)}


def _nll(pack, logprobs):
    mask = pack["packed_response_mask"].to(logprobs.dtype)
    return -(logprobs * mask).sum() / mask.sum().clamp_min(1), {"tokens": mask.sum()}


def test_packed_logprobs_equal_each_sequence_on_its_own():
    mgr, model = _manager()
    pack = _pack([9, 4, 12])
    packed = pack_train_data(pack)
    with torch.no_grad():
        lp = mgr.forward_logprobs(packed)
        assert lp.shape == (8 + 3 + 11,)
        k = 0
        for r, n in enumerate([9, 4, 12]):
            ids = pack["input_ids"][r, :n]
            h = model(ids, torch.arange(n), TrainMeta(build_varlen_meta([n]), False)).hidden_states
            want = torch.log_softmax(model.compute_logits(h).float(), -1)[:-1].gather(-1, ids[1:, None]).squeeze(-1)
            assert torch.allclose(lp[k:k + n - 1], want, atol=1e-5), r
            k += n - 1


def test_micro_batches_accumulate_into_one_update():
    packs = [_pack([9, 4], seed=1), _pack([12], seed=2), _pack([5, 6, 7], seed=3)]
    mgr, model = _manager(_nll)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    stats = mgr.train([dict(p) for p in packs])
    assert [s["stepped"] for s in stats] == [False, False, True] and [s["global_step"] for s in stats] == [0, 0, 1]
    assert [s["num_tokens"] for s in stats] == [13, 12, 18] and stats[-1]["metrics"]["grad_norm"] > 0
    assert "grad_norm" not in stats[0]["metrics"] and stats[0]["metrics"]["tokens"] == 7 + 2
    assert any(not torch.equal(before[n], p) for n, p in model.named_parameters())
    # the accumulated fp32 gradient buffers equal one backward pass through the mean of the three losses (compared
    # before the optimizer: Adam's first step turns rounding noise on near-zero gradients into full-size updates)
    acc_mgr, acc_model = _manager(_nll)
    for p in packs:
        acc_mgr.train_step(dict(p), allow_step=False, grad_scale=3)
    ref_mgr, ref_model = _manager(_nll)
    losses = []
    for p in packs:
        packed = pack_train_data(dict(p))
        losses.append(_nll(packed, ref_mgr.forward_logprobs(packed))[0])
    (sum(losses) / 3).backward()
    ref_mgr.optimizer.fold_param_grads()
    for (n, a), (_, b) in zip(acc_model.named_parameters(), ref_model.named_parameters()):
        assert torch.allclose(a.main_grad, b.main_grad, atol=1e-6), n
        assert a.grad is None and float(a.main_grad.abs().sum()) > 0
    assert [float(s["loss"]) for s in stats] == pytest.approx([float(x.detach()) for x in losses], rel=1e-5)


def test_accumulation_groups_step_at_their_last_micro_batch():
    mgr, _ = _manager(_nll)
    packs = [_pack([6, 5], seed=i) for i in range(5)]
    stats = mgr.train(packs, gradient_accumulation_steps=2)
    assert [s["stepped"] for s in stats] == [False, True, False, True, True]         # the tail group has one member
    assert [s["global_step"] for s in stats] == [0, 1, 1, 2, 3] and mgr.global_step == 3


def test_learning_rate_follows_the_schedule_per_optimizer_step():
    mgr, _ = _manager(_nll, lr=1e-2, min_lr=1e-3, lr_decay_style="linear", lr_decay_steps=4)
    stats = mgr.train([_pack([6], seed=i) for i in range(3)], gradient_accumulation_steps=1)
    assert [s["metrics"]["lr"] for s in stats] == pytest.approx([1e-2 - 9e-3 * k / 4 for k in (1, 2, 3)])


def test_the_loss_function_comes_from_the_pack_or_from_the_manager():
    mgr, _ = _manager()
    with pytest.raises(ValueError, match="no loss function"):
        mgr.train([_pack([6])])
    pack = _pack([6])
    pack["_loss_fn"] = lambda p, lp: lp.sum() * 0.0 + 3.0          # a bare tensor is a valid return value
    out = mgr.train([pack])
    assert out[0]["loss"] == 3.0 and out[0]["stepped"] and set(out[0]["metrics"]) == {"lr", "grad_norm"}
    bad = _pack([6])
    bad["_loss_fn"] = lambda p, lp: 1.0
    with pytest.raises(TypeError, match="must return a torch.Tensor"):
        mgr.train([bad])


def test_per_rank_shards_are_selected_by_the_data_parallel_rank():
    mgr, _ = _manager(_nll)
    mine, other = _pack([6, 4], seed=1), None
    out = mgr.train([[mine, other]])                  # a list per micro-batch: one entry per data-parallel rank
    assert out[0]["num_tokens"] == 10
