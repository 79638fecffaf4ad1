"""``--tune-params`` search logic on CPU with scripted probes: which candidates exist, in which order they are probed,
what ends a stage, which errors count as "does not fit", and what the probes feed the trainer."""

from __future__ import annotations

import logging

import pytest
import torch

from areno_b200.api.trainer_config import PolicyTrainerConfig, TrainerConfig
from areno_b200.cli import auto_tune as at


def _cfg(**kw):
    base = dict(algo="gspo", ckpt="m", dataset_path="d", batch_size=32, n_samples=8, mini_bs=16)
    base.update(kw)
    return PolicyTrainerConfig(**base)


def _fits(limit_rollout: int, limit_mini: int):
    """Probe whose memory use grows with concurrency / micro-batch size; records every call."""
    calls = []

    def probe(config, cand, stage):
        calls.append((stage, cand))
        size, limit = (cand.max_running_prompts, limit_rollout) if stage == "rollout" else (cand.mini_bs, limit_mini)
        return at.AutoTuneMeasurement(cand, min(1.0, 0.5 * size / limit), ok=True)

    return probe, calls


@pytest.mark.parametrize("value,expect", [(0, [1]), (1, [1]), (2, [1, 2]), (300, [1, 2, 4, 8, 16, 32, 64, 128, 256])])
def test_powers_of_two_cover_the_range(value, expect):
    assert at.powers_of_two_up_to(value) == expect


def test_sparse_select_keeps_both_ends_and_order():
    items = list(range(40))
    picked = at.sparse_select(items, 6)
    assert picked[0] == 0 and picked[-1] == 39 and picked == sorted(picked) and len(picked) == 6
    assert at.sparse_select(items, 100) == items and at.sparse_select(items, 1) == [39]


def test_rollout_candidates_are_largest_first_and_bounded_by_the_sample_cap():
    cands = at.rollout_candidates(_cfg(), auto_max_samples=48)
    assert [c.max_running_prompts for c in cands] == [32, 16, 8, 4, 2, 1]
    assert all(c.tp_size == _cfg().tp_size and c.n_samples == 8 and not c.keep_rollout_state for c in cands)
    many = at.rollout_candidates(_cfg(), auto_max_samples=1 << 20)
    assert len(many) == 16 and many[0].max_running_prompts == 1 << 20 and many[-1].max_running_prompts == 1


def test_train_template_derives_the_batch_from_the_rollout_concurrency():
    ro = at.rollout_candidates(_cfg(n_samples=8), auto_max_samples=256)[2]          # 64 concurrent rows
    t = at.train_template(_cfg(n_samples=8), ro, auto_max_samples=256)
    assert (t.batch_size, t.n_samples, t.train_rows, t.mini_bs) == (8, 8, 64, 16)
    # fewer rows than samples per prompt still gives one prompt
    small = at.train_template(_cfg(n_samples=8), at.rollout_candidates(_cfg(), auto_max_samples=4)[0], auto_max_samples=4)
    assert small.batch_size == 1 and small.mini_bs <= small.train_rows


def test_train_candidates_vary_batch_and_micro_batch_within_limits():
    template = at.train_template(_cfg(), at.rollout_candidates(_cfg(), auto_max_samples=256)[0], auto_max_samples=256)
    cands = at.train_candidates(_cfg(mini_bs=8), template, auto_max_samples=64)
    assert {c.n_samples for c in cands} == {8} and max(c.batch_size for c in cands) == 8      # 64 rows / 8 samples
    assert max(c.mini_bs for c in cands) == 8 and all(c.mini_bs <= c.train_rows for c in cands)
    assert cands == sorted(cands, key=lambda c: (c.train_rows, c.mini_bs)) and len(cands) <= 32


def test_user_tp_size_and_adam_choice_are_carried_through_unchanged():
    probe, calls = _fits(64, 4)
    res = at.auto_tune_config(_cfg(tp_size=2, adam_8bit=True), mem_frac=0.9, probe_fn=probe)
    assert {c.tp_size for _s, c in calls} == {2} and {c.adam_8bit for _s, c in calls} == {True}
    assert res.config.tp_size == 2 and res.config.adam_8bit is True


def test_largest_fitting_candidate_wins_each_stage():
    probe, calls = _fits(limit_rollout=64, limit_mini=4)
    res = at.auto_tune_config(_cfg(), mem_frac=0.6, auto_max_samples=256, probe_fn=probe)
    ro = [c.max_running_prompts for s, c in calls if s == "rollout"]
    tr = [c.mini_bs for s, c in calls if s == "train"]
    assert ro == [256, 128, 64] and tr == [16, 8, 4]                # stops at the first that fits
    assert (res.config.max_running_prompts, res.config.mini_bs, res.config.batch_size) == (64, 4, 8)
    assert res.measurement.peak_mem_frac == 0.5 and len(res.measurements) == 6


def test_explicit_concurrency_skips_the_rollout_stage():
    probe, calls = _fits(64, 16)
    res = at.auto_tune_config(_cfg(max_running_prompts=24), mem_frac=0.9, probe_fn=probe)
    assert all(stage == "train" for stage, _c in calls)
    assert res.config.max_running_prompts == 24 and res.config.batch_size == 2       # floor_pow2(24 // 8)


def test_progress_is_logged_per_probe(caplog):
    probe, _calls = _fits(256, 16)
    with caplog.at_level(logging.INFO, logger=at.logger.name):
        at.auto_tune_config(_cfg(), mem_frac=0.9, auto_max_samples=8, probe_fn=probe)
    text = caplog.text
    assert "auto tune rollout probe 1/4" in text and "auto tune train probe 1/" in text and "auto tune selected" in text


def test_nothing_fits_is_an_error_that_quotes_the_first_failure():
    def probe(config, cand, stage):
        return at.AutoTuneMeasurement(cand, 1.0, ok=False, error="CUDA out of memory while probing")

    with pytest.raises(RuntimeError, match="rollout stage could not find a candidate.*CUDA out of memory while probing"):
        at.auto_tune_config(_cfg(), probe_fn=probe)


@pytest.mark.parametrize("kwargs,msg", [(dict(mem_frac=0.0), "mem-frac"), (dict(mem_frac=1.5), "mem-frac"),
                                         (dict(auto_max_samples=0), "tune-max-samples")])
def test_arguments_are_validated(kwargs, msg):
    with pytest.raises(ValueError, match=msg):
        at.auto_tune_config(_cfg(), probe_fn=lambda *a: None, **kwargs)


def test_offline_trainers_are_refused():
    sft = TrainerConfig(algo="sft", ckpt="m", dataset_path="d")
    with pytest.raises(ValueError, match="rollout-based trainers only"):
        at.auto_tune_config(sft, probe_fn=lambda *a: None)


@pytest.mark.parametrize("message,oom", [
    ("CUDA out of memory. Tried to allocate 2.00 GiB", True),
    ("worker exited without reporting result (exitcode -9) during Op.TRAIN", True),
    ("worker exited without reporting result during Op.PROBE_ROLLOUT_CACHE", True),
    ("worker rank 3 failed during Op.PROBE_ROLLOUT_CACHE: NCCL error: unhandled system call failure", True),
    ("worker rank 3 failed during Op.TRAIN: NCCL error", False),
    ("worker exited without reporting result (exitcode 1) during Op.SAVE_CHECKPOINT", False),
    ("tokenizer file missing", False)])
def test_which_failures_count_as_out_of_memory(message, oom):
    assert at.is_oom_error(message) is oom


def test_probe_wrapper_turns_memory_and_tp_errors_into_rejections(monkeypatch):
    cand = at.rollout_candidates(_cfg(), auto_max_samples=4)[0]

    def boom(exc):
        def run(config, candidate, *, stage):
            raise exc
        return run

    monkeypatch.setattr(at, "_run_dummy_probe", boom(RuntimeError("CUDA out of memory")))
    m = at.probe_candidate_with_dummy_run(_cfg(), cand, "rollout")
    assert not m.ok and m.peak_mem_frac == 1.0 and "out of memory" in m.error
    monkeypatch.setattr(at, "_run_dummy_probe", boom(ValueError("num_attention_heads=28 must be divisible by tp_size=8")))
    assert not at.probe_candidate_with_dummy_run(_cfg(), cand, "train").ok
    monkeypatch.setattr(at, "_run_dummy_probe", boom(RuntimeError("checkpoint not found")))
    with pytest.raises(RuntimeError, match="checkpoint not found"):
        at.probe_candidate_with_dummy_run(_cfg(), cand, "train")


@pytest.mark.parametrize("prompt,new,ctx,expect", [(512, 512, None, (512, 512)), (1024, 3071, 2048, (1024, 1024)),
                                                   (4096, 100, 2048, (2047, 1)), (0, 0, None, (1, 1))])
def test_probe_token_budgets_respect_the_context_limit(prompt, new, ctx, expect):
    assert at.dummy_token_budgets(max_prompt_tokens=prompt, max_new_tokens=new, max_context_len=ctx) == expect


def test_probe_rows_are_full_length_and_only_the_response_is_trained():
    rows = at.dummy_train_rows(prompt_tokens=[5, 6, 7], response_tokens=[8, 9], eos_token_id=2, target_rows=4)
    assert len(rows) == 4 and rows[0].tokens == [5, 6, 7, 8, 9]
    assert rows[0].prompt_mask == [True, True, True, False, False] and rows[0].loss_mask == [False] * 3 + [True] * 2
    assert rows[0].advantages == [0.0, 0.0, 0.0, 1.0, 1.0] and rows[0].eos_token_id == 2
    assert len(at.dummy_train_rows(prompt_tokens=[1], response_tokens=[2], eos_token_id=0, target_rows=0)) == 1


def test_filler_tokens_repeat_the_encoding_to_the_requested_width():
    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [11, 12, 13]

    assert at._filler_tokens(Tok(), 7, "x") == [11, 12, 13, 11, 12, 13, 11]

    class Broken:
        def encode(self, *a, **k):
            raise RuntimeError("no vocabulary")

    assert at._filler_tokens(Broken(), 3, "x") == [1, 1, 1]


def test_probe_loss_is_the_masked_mean_negative_logprob_and_differentiable():
    ids = torch.tensor([[1, 2, 3, 4]])
    pack = dict(input_ids=ids, lengths=torch.tensor([4]), prompt_mask=torch.tensor([[True, True, False, False]]),
                logprobs=torch.zeros(1, 4), advantages=torch.zeros(1, 4))
    lp = torch.tensor([[-0.5, -1.0, -2.0]], requires_grad=True)           # entry i is the log-prob of token i + 1
    loss, metrics = at.dummy_policy_loss(pack, lp)
    assert loss.item() == pytest.approx(1.5) and metrics["loss"].item() == pytest.approx(1.5)   # tokens 3 and 4: -(-1 - 2) / 2
    loss.backward()
    assert lp.grad is not None and lp.grad[0, 0] == 0 and lp.grad[0, 1] < 0


def test_summary_line_reports_the_choice():
    probe, _ = _fits(256, 16)
    res = at.auto_tune_config(_cfg(), mem_frac=0.9, auto_max_samples=16, probe_fn=probe)
    line = at.format_auto_tune_summary(res)
    assert "max_running_prompts=16" in line and "peak_mem_frac=" in line and "drop_rollout_state=True" in line
    assert at.format_auto_tune_summary(at.AutoTuneResult(res.config, None, ())) is None
