"""Spawned cluster on CPU (gloo): request routing over data-parallel ranks, error propagation with
the worker's traceback, and detection of a worker that dies between steps.  All failures are made on
the host (an exception raised by an op, a process that exits); no device is involved."""

from __future__ import annotations

import os
import signal
import time

import pytest
import torch

from areno_b200.engine.api import ArenoEngine
from areno_b200.engine.cluster import WorkerError
from areno_b200.engine.config import OptimizerConfig, RuntimeConfig
from areno_b200.engine.inference import SamplingParams
from areno_b200.engine.protocol import Op

from .helpers import tiny_config


def _engine(dp=2, **kw):
    return ArenoEngine.from_pretrained(
        None, model_config=tiny_config(), tp_size=1, dp_size=dp, devices=list(range(dp)), dummy_load=True, backend="gloo",
        launcher="spawn", seed=2, optimizer_config=OptimizerConfig(lr=1e-2, weight_decay=0.0),
        runtime_config=RuntimeConfig(eager_decode=True, max_model_len=128, activation_checkpointing=False),
        max_running_seqs=4, **kw)


def _loss(pack, logprobs):
    from areno_b200.api.loss_fns import grpo_loss_fn

    return grpo_loss_fn(pack, logprobs)


def _broken_loss(pack, logprobs):
    raise RuntimeError("loss function exploded on purpose")


def _pack(prompt, toks, lps):
    n = len(prompt) + len(toks)
    pm = torch.ones((1, n), dtype=torch.bool)
    pm[0, len(prompt):] = False
    lp = torch.zeros((1, n))
    lp[0, len(prompt):] = torch.tensor(lps)
    adv = torch.zeros((1, n))
    adv[0, len(prompt):] = 1.0
    return dict(input_ids=torch.tensor([prompt + toks]), lengths=torch.tensor([n]), prompt_mask=pm, logprobs=lp,
                advantages=adv)


@pytest.mark.timeout(300)
def test_rollout_and_step_over_two_dp_ranks_then_failures():
    eng = _engine()
    try:
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(3, 512, (n,), generator=g).tolist() for n in (12, 30, 7, 19, 25)]
        out = eng.generate_rollout(prompts, max_new_tokens=5, max_running_prompts=8,
                                   sampling_params=SamplingParams(temperature=0.0))
        assert [len(t) for t in out.tokens] == [5] * 5          # merged back in input order over both ranks
        info = eng.model_info()
        assert info["dp_size"] == 2 and info["vocab_size"] == 512
        # both ranks hold the same weights, so greedy decoding of a prompt is rank-independent
        again = eng.generate_rollout(list(reversed(prompts)), max_new_tokens=5, max_running_prompts=8,
                                     sampling_params=SamplingParams(temperature=0.0))
        assert list(reversed(again.tokens)) == out.tokens
        packs =[_pack(p, t, l) for p, t, l in zip(prompts[:4], out.tokens, out.logprobs)]
        for pk in packs:
            pk["_loss_fn"] = _loss
        stats = eng.step([{k: (torch.cat([a[k], b[k]], 0) if k != "_loss_fn" and a[k].shape[1:] == b[k].shape[1:] else a[k])
                           for k in a} for a, b in zip(packs[:1], packs[:1])])
        assert stats and stats[-1]["stepped"]

        # 1. an exception inside a worker op comes back as WorkerError carrying the remote traceback,
        #    and the cluster keeps serving afterwards
        bad = dict(packs[0])
        bad["_loss_fn"] = _broken_loss
        with pytest.raises(WorkerError, match="loss function exploded on purpose"):
            eng.step([{k: (torch.cat([v, v], 0) if isinstance(v, torch.Tensor) else v) for k, v in bad.items()}])
        assert eng.model_info()["dp_size"] == 2

        # 2. a worker that exits between steps is noticed by the result pump: the next call fails fast
        victim = eng.cluster._procs[1]
        os.kill(victim.pid, signal.SIGKILL)
        victim.join(timeout=10)
        t0 = time.time()
        with pytest.raises(WorkerError, match="exited without reporting"):
            eng.cluster.call(Op.MODEL_INFO, None, timeout=60)
        assert time.time() - t0 < 30
    finally:
        eng.close()


@pytest.mark.timeout(300)
def test_samples_of_one_prompt_differ_across_data_parallel_ranks():
    """The samples of a prompt are dealt over both ranks, which share a seed and number their requests alike: sampled
    (not greedy) completions must still all differ instead of coming out in identical pairs."""
    eng = _engine()
    try:
        prompt = torch.randint(3, 512, (12,), generator=torch.Generator().manual_seed(0)).tolist()
        group = eng.generate_rollout([prompt] * 4, max_new_tokens=8, max_running_prompts=8,
                                     sampling_params=SamplingParams(temperature=1.0))
        assert len({tuple(t) for t in group.tokens}) == 4
        seeded = [eng.generate_rollout([prompt] * 4, max_new_tokens=8, max_running_prompts=8,
                                       sampling_params=SamplingParams(temperature=1.0, seed=21)).tokens for _ in range(2)]
        assert seeded[0] == seeded[1] and len({tuple(t) for t in seeded[0]}) == 4
        # role scoring: rows are dealt over the ranks by stride and come back in row order; a frozen reference built
        # from the actor's weights scores exactly like the actor
        from areno_b200.api.roles import ModelRole

        g = torch.Generator().manual_seed(1)
        rows = [torch.randint(3, 512, (n,), generator=g).tolist() for n in (9, 4, 12, 7, 5)]
        eng.ensure_roles({"ref": ModelRole("ref", "", trainable=False), "critic": ModelRole("critic", "", trainable=True)})
        ref, actor = eng.score_logprobs("ref", rows), eng.score_logprobs("actor", rows)
        assert [len(r) for r in ref] == [len(r) for r in rows] and all(r[0] == 0.0 and max(r[1:]) < 0 for r in ref)
        for a, b in zip(ref, actor):
            assert a == pytest.approx(b, abs=1e-6)
        assert eng.score_logprobs("ref", list(reversed(rows)))[0] == pytest.approx(ref[-1], abs=1e-6)
        values = eng.score_values("critic", rows)
        assert [len(v) for v in values] == [len(r) for r in rows] and all(x == 0.0 for v in values for x in v)   # zero head
    finally:
        eng.close()


def _sleepy_loss(pack, logprobs):
    time.sleep(300)
    return logprobs.sum()


@pytest.mark.timeout(180)
def test_watchdog_stops_the_workers_of_a_call_that_runs_past_its_deadline(monkeypatch):
    monkeypatch.setenv("ARENO_OP_DEADLINE_S", "600")               # read at construction; tightened below
    eng = _engine(dp=1)
    try:
        assert eng.cluster.op_deadline_s == 600.0
        prompt = list(range(3, 12))
        out = eng.generate_rollout([prompt], max_new_tokens=3, max_running_prompts=2,
                                   sampling_params=SamplingParams(temperature=0.0))
        pack = _pack(prompt, out.tokens[0], out.logprobs[0])
        pack["_loss_fn"] = _sleepy_loss
        procs = list(eng.cluster._procs)
        eng.cluster.op_deadline_s = 2.0
        t0 = time.time()
        with pytest.raises(WorkerError, match=r"not answered within the 2 s deadline by rank\(s\) \[0\]"):
            eng.step([pack])
        assert time.time() - t0 < 60
        assert all(not p.is_alive() for p in procs)                # processes stopped; nothing else was touched
        with pytest.raises(WorkerError, match="closed"):
            eng.cluster.call(Op.MODEL_INFO)
    finally:
        eng.close()


@pytest.mark.timeout(120)
def test_start_up_failure_is_reported():
    cfg = tiny_config(num_attention_heads=4, num_key_value_heads=2)
    with pytest.raises((WorkerError, ValueError)):
        ArenoEngine.from_pretrained("/nonexistent/model/dir", model_config=cfg, tp_size=1, dp_size=1, devices=[0],
                                    backend="gloo", launcher="spawn",
                                    runtime_config=RuntimeConfig(eager_decode=True, max_model_len=64))
