"""CPU-side helpers of the benchmark script: synthetic prompts and rewards are reproducible, micro-batches respect the
token cap, clock samples are summarised the way the result line reports them, and the argument surface the driver uses
exists."""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_synthetic_prompts_and_rewards_are_reproducible_and_rank_specific():
    b = _bench()
    a = b.make_prompts(3, 0, 1000, 8, 16, 64)
    assert a == b.make_prompts(3, 0, 1000, 8, 16, 64) and a != b.make_prompts(3, 1, 1000, 8, 16, 64)
    assert a != b.make_prompts(4, 0, 1000, 8, 16, 64)
    assert len(a) == 8 and all(16 <= len(p) <= 64 and all(3 <= t < 1000 for t in p) for p in a)
    rewards = [b.hash_reward(p) for p in b.make_prompts(0, 0, 50000, 200, 4, 12)]
    assert set(rewards) == {0.0, 1.0} and 60 < sum(rewards) < 140                  # a fair coin over token hashes
    assert b.hash_reward([1, 2, 3]) == b.hash_reward([1, 2, 3])


def test_group_advantages_standardise_within_each_prompts_samples():
    b = _bench()
    adv = b.group_advantages(np.array([1.0, 0.0, 1.0, 0.0, 1.0, 1.0, 1.0, 1.0]), 4)
    assert np.allclose(adv[:4], [1, -1, 1, -1], atol=1e-4) and np.allclose(adv[4:], 0.0)


def test_micro_batches_respect_the_token_cap_and_given_groups():
    b = _bench()
    prompts = [[1] * n for n in (30, 40, 50, 20)]
    responses = [[2] * 10] * 4
    logprobs = [[-0.5] * 10] * 4
    packs = b.build_micro_batches(prompts, responses, logprobs, [1.0, -1.0, 0.5, 0.0], micro_tokens=100)
    assert [p["lengths"].tolist() for p in packs] == [[40, 50], [60, 30]]
    first = packs[0]
    assert first["input_ids"].shape == (2, 50) and first["prompt_mask"][0, :30].all() and not first["prompt_mask"][0, 30:40].any()
    assert first["prompt_mask"][0, 40:].all()                                        # padding counts as prompt
    assert first["advantages"][1, 40:50].tolist() == [-1.0] * 10 and float(first["logprobs"][0, 29]) == 0.0
    grouped = b.build_micro_batches(prompts, responses, logprobs, [0.0] * 4, micro_tokens=1, groups=[[3, 0], [1], [2]])
    assert [p["lengths"].tolist() for p in grouped] == [[30, 40], [50], [60]]


def test_clock_samples_are_summarised_as_median_clock_and_active_reasons():
    b = _bench()
    s = b.ClockSampler(0)
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"]

    class Done:
        def terminate(self):
            pass

    s.proc = Done()
    s.lines = ["0, 1800, 1965, 950.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1900, 1965, 900.0, 0x0, Not Active, Not Active, Not Active, Not Active",
               "0, 1700, 1965, 990.0, 0x4, Not Active, Active, Not Active, Active",
               "garbage", "0, [N/A], 1965, 1, 0, a, b, c, d"]
    out = s.stop()
    assert out == {"sm_mhz": 1800.0, "sm_max_mhz": 1965.0, "reasons": ["hw_thermal_slowdown", "sw_power_cap"], "samples": 3}
    s.lines = []
    assert s.stop()["reasons"] == ["no samples"]


def test_argument_surface_of_the_driver_contract(monkeypatch):
    b = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = b.parse_args()
    assert args.gpus == 1 and args.warmup >= 3 and args.steps >= 1 and args.impl in ("ours", None, "areno_b200")
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "8", "--steps", "5", "--warmup", "4", "--impl", "reference"])
    args = b.parse_args()
    assert (args.gpus, args.steps, args.warmup, args.impl) == (8, 5, 4, "reference")
    assert b.pick_rollout_tp(8) in (1, 2, 4, 8) and b.pick_rollout_tp(1) == 1
    monkeypatch.setenv("ARENO_BENCH_ROLLOUT_TP", "4")
    assert b.pick_rollout_tp(8) == 4 and b.pick_rollout_tp(6) == 1                   # must divide the world
