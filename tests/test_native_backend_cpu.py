"""The native backend of the SDK against a scripted engine, on the CPU: ragged rows padded into training packs, what
a rollout request turns into (EOS, stop and suppressed ids, greedy), samples grouped back per prompt, how per-micro-batch
statistics become one training result, and argument checks."""

from __future__ import annotations

import asyncio
from functools import partial
from types import SimpleNamespace

import pytest
import torch

from areno_b200.api import ArenoConfig
from areno_b200.api.backend.native import (NativeBackend, explicit_suppress_token_ids, make_train_pack, pad_rows,
                                           pad_token_id, rollout_options)
from areno_b200.api.loss_fns import grpo_loss_fn, sft_loss_fn
from areno_b200.api.models import SamplingParams, TrainSequence
from tests.helpers import FakeTokenizer


def _ctx(**kw):
    base = dict(tokenizer=FakeTokenizer(), eos_token_ids=(2,), custom_config=ArenoConfig(tp_size=1), world_size=1,
                model_path="m")
    base.update(kw)
    return SimpleNamespace(**base)


class ScriptedEngine:
    def __init__(self):
        self.calls = []
        self.config = SimpleNamespace(dp_size=4, model=SimpleNamespace(max_position_embeddings=4096))

    def generate_rollout(self, prompts, **kw):
        self.calls.append(("rollout", prompts, kw))
        return SimpleNamespace(tokens=[[len(p), i] for i, p in enumerate(prompts)],
                               logprobs=[[-1.0, -float(i)] for i in range(len(prompts))])

    async def generate_rollout_async(self, prompts, **kw):
        self.calls.append(("rollout_async", prompts, kw))
        return SimpleNamespace(tokens=[[7] for _ in prompts], logprobs=[[-0.5] for _ in prompts])

    def step(self, packs, gradient_accumulation_steps=None, local=False):
        self.calls.append(("step", packs, gradient_accumulation_steps, local))
        return [{"loss": float(i), "global_step": 10 + i,
                 "metrics": {"ratio_mean": 1.0 + i, "lr": 0.1 * (i + 1), "grad_norm": 2.0 * (i + 1), "kl": float(i), "tag": "x"}}
                for i, _ in enumerate(packs)]

    def train_values(self, role, packs, **kw):
        self.calls.append(("train_values", role, len(packs), kw))
        return {"value_loss": 0.5}

    def score_logprobs(self, role, rows, pad_token_id=0, microbatch_size=8):
        return [("lp", role, pad_token_id, microbatch_size)] * len(rows)

    def score_values(self, role, rows, pad_token_id=0):
        return [("v", pad_token_id)] * len(rows)

    def score_rewards(self, role, rows, pad_token_id=0):
        return [("r", pad_token_id)] * len(rows)

    def ensure_roles(self, roles):
        self.calls.append(("roles", roles))

    def save_checkpoint(self, path):
        return path

    def probe_rollout_cache(self, **kw):
        return 0.4

    def close(self):
        self.calls.append(("close",))


# ------------------------------------------------------------------------------------------------------ packing

def test_ragged_rows_are_right_padded_and_cut_to_the_width():
    out = pad_rows([[1, 2, 3], [], [4]], dtype=torch.long, fill_value=9)
    assert out.tolist() == [[1, 2, 3], [9, 9, 9], [4, 9, 9]] and out.dtype == torch.long
    assert pad_rows([[1, 2, 3], [4]], dtype=torch.int32, width=2).tolist() == [[1, 2], [4, 0]]
    assert pad_rows([[True], [False, True]], dtype=torch.bool, fill_value=True).tolist() == [[True, True], [False, True]]
    assert pad_rows([[0.5]], dtype=torch.float32, width=3).tolist() == [[0.5, 0.0, 0.0]]
    assert pad_rows([], dtype=torch.long).shape == (0, 0) and pad_rows([[], []], dtype=torch.long).shape == (2, 0)


def test_training_pack_layout():
    a = TrainSequence(tokens=[5, 6, 7, 8], prompt_mask=[True, True, False, False], logprobs=[0, 0, -1.0, -2.0],
                      advantages=[0, 0, 1.0, 1.0], eos_token_id=2)
    b = TrainSequence(tokens=[9, 10], prompt_mask=[True, False], logprobs=[0, -0.5], advantages=[0, -1.0], eos_token_id=2)
    pack = make_train_pack([a, b])
    assert pack["input_ids"].tolist() == [[5, 6, 7, 8], [9, 10, 2, 2]] and pack["lengths"].tolist() == [4, 2]
    assert pack["prompt_mask"].tolist() == [[True, True, False, False], [True, False, True, True]]     # padding is "prompt"
    assert pack["logprobs"][1].tolist() == [0, -0.5, 0, 0] and pack["advantages"][1].tolist() == [0, -1.0, 0, 0]
    assert torch.equal(pack["labels"], pack["input_ids"]) and pack["labels"] is not pack["input_ids"]
    assert not {"loss_mask", "returns", "values", "ref_logprobs"} & set(pack)
    with pytest.raises(ValueError, match="empty"):
        make_train_pack([])


def test_optional_signals_appear_when_any_sequence_has_them():
    a = TrainSequence(tokens=[1, 2, 3], prompt_mask=[True, False, False], loss_mask=[False, True, False],
                      ref_logprobs=[0, -1.0, -1.0], logprobs=[0, 0, 0], advantages=[0, 0, 0])
    b = TrainSequence(tokens=[4, 5], prompt_mask=[True, False], logprobs=[0, 0], advantages=[0, 0], values=[0.1, 0.2],
                      returns=[1.0, 1.0])
    pack = make_train_pack([a, b])
    assert pack["loss_mask"].tolist() == [[False, True, False], [False, True, False]]    # b falls back to "not prompt"
    assert pack["ref_logprobs"].tolist() == [[0, -1.0, -1.0], [0, 0, 0]]
    assert pack["values"].shape == (2, 3) and pack["returns"][1].tolist() == [1.0, 1.0, 0.0]


# ------------------------------------------------------------------------------------------------------ rollout

def test_rollout_options_from_tokenizer_and_sampling_parameters():
    ctx = _ctx()
    opts = rollout_options(ctx, SamplingParams(temperature=0.7, top_p=0.9, top_k=-1, stop_token_ids=[40], max_prompt_len=99))
    sp = opts["sampling_params"]
    assert opts["eos_token_id"] == (2,) and opts["max_prompt_len"] == 99
    assert (sp.temperature, sp.top_p, sp.top_k, sp.stop_token_ids) == (0.7, 0.9, 0, (40,))
    assert sp.suppress_token_ids == (0, 1)                   # pad and bos may never be sampled; EOS may
    assert sp.seed is None and sp.min_new_tokens == 0
    seeded = rollout_options(ctx, SamplingParams(seed=17, min_new_tokens=3))["sampling_params"]
    assert seeded.seed == 17 and seeded.min_new_tokens == 3
    greedy = rollout_options(ctx, SamplingParams(greedy=True, temperature=0.9, ignore_eos=True))
    assert greedy["sampling_params"].temperature == 0.0 and greedy["eos_token_id"] == ()
    assert greedy["sampling_params"].suppress_token_ids == (0, 1)
    assert explicit_suppress_token_ids(SimpleNamespace(pad_token_id=3, bos_token_id=3, unk_token_id=True)) == (3,)
    no_tok = rollout_options(_ctx(tokenizer=None), SamplingParams())
    assert no_tok["sampling_params"].suppress_token_ids == ()
    with pytest.raises(TypeError, match="ArenoConfig"):
        rollout_options(_ctx(custom_config={"tp_size": 1}), SamplingParams())


def test_samples_are_grouped_per_prompt_in_request_order():
    eng = ScriptedEngine()
    backend = NativeBackend(engine=eng)
    results = backend.rollout_batch(_ctx(), [[1, 2, 3], [4]], 2, SamplingParams(max_new_tokens=5))
    kind, flat, kw = eng.calls[0]
    assert flat == [[1, 2, 3], [1, 2, 3], [4], [4]] and kw["max_new_tokens"] == 5 and kw["local"] is False
    assert [[s.resp_tokens for s in r.sequences] for r in results] == [[[3, 0], [3, 1]], [[1, 2], [1, 3]]]
    assert results[1].sequences[1].resp_logprobs == [-1.0, -3.0]
    out = asyncio.run(backend.rollout_batch_async(_ctx(), [[1]], 3, SamplingParams()))
    assert len(out) == 1 and len(out[0].sequences) == 3 and eng.calls[1][0] == "rollout_async"
    local = _ctx(custom_config=ArenoConfig(tp_size=1, spmd_local_data=True))
    backend.rollout_batch(local, [[1]], 1, SamplingParams())
    assert eng.calls[2][2]["local"] is True


# -------------------------------------------------------------------------------------------------------- train

def _seqs(n):
    return [TrainSequence(tokens=[1, 2, 3 + i], prompt_mask=[True, False, False], logprobs=[0, -1.0, -1.0],
                          advantages=[0, 1.0, 1.0]) for i in range(n)]


def test_train_cuts_micro_batches_and_reduces_their_statistics():
    eng = ScriptedEngine()
    backend = NativeBackend(engine=eng)
    res = backend.train(_ctx(), _seqs(5), grpo_loss_fn, mini_bs=2, gradient_accumulation_steps=3)
    _, packs, accum, local = eng.calls[0]
    assert [p["input_ids"].shape[0] for p in packs] == [2, 2, 1] and accum == 3 and not local
    assert all(p["_loss_fn"] is grpo_loss_fn and "_sft_total_target_tokens" not in p for p in packs)
    assert res["loss"] == 1.0 and res["num_microbatches"] == 3 and res["global_step"] == 12
    assert res["ratio_mean"] == 1.0                       # from the first micro-batch: before this step's updates
    assert res["lr"] == pytest.approx(0.3) and res["grad_norm"] == 6.0      # from the last one
    assert res["kl"] == 1.0 and "tag" not in res and res["backend_train_time_s"] >= 0
    with pytest.raises(ValueError, match="empty"):
        backend.train(_ctx(), [], grpo_loss_fn, mini_bs=2)
    assert NativeBackend._reduce_stats([], 0.0) == {}


def test_sft_training_annotates_the_token_mean_over_the_accumulation_group():
    eng = ScriptedEngine()
    backend = NativeBackend(engine=eng)
    for fn in (sft_loss_fn, partial(sft_loss_fn)):
        backend.train(_ctx(), _seqs(3), fn, mini_bs=2, gradient_accumulation_steps=None)
        packs = eng.calls[-1][1]
        assert [p["_sft_total_target_tokens"] for p in packs] == [6, 6] and packs[0]["_sft_grad_scale"] == 2


def test_roles_scoring_and_housekeeping_pass_through_with_the_pad_token():
    eng = ScriptedEngine()
    backend = NativeBackend(engine=eng)
    ctx = _ctx()
    assert backend.score_logprobs(ctx, "ref", [[1], [2]], microbatch_size=4) == [("lp", "ref", 0, 4)] * 2
    assert backend.score_values(ctx, "critic", [[1]]) == [("v", 0)] and backend.score_rewards(ctx, "rm", [[1]]) == [("r", 0)]
    assert pad_token_id(_ctx(tokenizer=SimpleNamespace(pad_token_id=None, eos_token_id=7))) == 7
    assert pad_token_id(_ctx(tokenizer=SimpleNamespace(pad_token_id=None, eos_token_id=None), eos_token_ids=(11,))) == 11
    assert backend.train_values(ctx, "critic", _seqs(3), 2, cliprange_value=0.2) == {"value_loss": 0.5}
    assert eng.calls[-1] == ("train_values", "critic", 2, {"gradient_accumulation_steps": None, "cliprange_value": 0.2,
                                                           "value_loss_coef": 0.5})
    assert backend.dp_size(ctx) == 4 and backend.model_context_len(ctx) == 4096
    assert backend.save_checkpoint(ctx, "/tmp/out") == "/tmp/out"
    assert backend.probe_rollout_cache(ctx, max_new_tokens=1, max_running_prompts=1, max_prompt_len=1) == 0.4
    backend.close()
    backend.close()
    assert eng.calls.count(("close",)) == 1
    with pytest.raises(RuntimeError, match="not initialized"):
        backend.dp_size(ctx)


def test_initialisation_checks_the_layout_before_building_an_engine():
    with pytest.raises(TypeError, match="ArenoConfig"):
        NativeBackend().initialize(_ctx(custom_config=object()))
    with pytest.raises(ValueError, match="divisible by tp_size"):
        NativeBackend().initialize(_ctx(world_size=3, custom_config=ArenoConfig(tp_size=2)))
    with pytest.raises(ValueError, match="must equal world_size"):
        NativeBackend().initialize(_ctx(world_size=4, custom_config=ArenoConfig(tp_size=2, dp_size=3)))
