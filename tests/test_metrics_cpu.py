"""Scalar channels of the metrics recorder on the CPU: which tags a training step writes and with what values.
Behaviours follow the reference's ``tests/test_metrics_cpu.py``."""

from __future__ import annotations

import pytest

from areno_b200.api import metrics
from areno_b200.api.models import TrainSequence


class RecordingWriter:
    def __init__(self):
        self.scalars, self.flushed, self.closed = {}, 0, 0

    def add_scalar(self, tag, value, step):
        self.scalars[tag] = (float(value), step)

    def flush(self):
        self.flushed += 1

    def close(self):
        self.closed += 1


def _batch():
    return [TrainSequence(tokens=[1, 2, 3, 4], prompt_mask=[True, True, False, False], logprobs=[9, 9, -1.0, -2.0],
                          advantages=[9, 9, 1.0, 1.0], reward=1.0),
            TrainSequence(tokens=[1, 2, 3], prompt_mask=[True, False, False], logprobs=[9, -1.0, -0.5],
                          advantages=[9, -1.0, -1.0], reward=0.0)]


def test_batch_statistics_leave_out_prompt_positions():
    stats = metrics.collect_train_batch_stats(_batch())
    assert stats["rewards"] == [1.0, 0.0] and stats["logprobs"] == [-1.0, -2.0, -1.0, -0.5]
    assert stats["advantages"] == [1.0, 1.0, -1.0, -1.0]
    assert stats["prompt_len"] == [2, 1] and stats["response_len"] == [2, 2] and stats["seq_len"] == [4, 3]
    assert stats["skipped_long"] == 0 and stats["total_skipped_long"] == 0


def test_rollout_statistics_keep_their_skip_counters():
    stats = metrics.init_rollout_stats(skipped_long=3, total_skipped_long=11)
    metrics.record_rollout_sequence_stats(stats, prefix_len=5, response_logprobs=[-0.5, -0.25], response_len=2)
    assert stats["skipped_long"] == 3 and stats["total_skipped_long"] == 11
    assert stats["seq_len"] == [7] and stats["logprobs"] == [-0.5, -0.25] and stats["rewards"] == []


def test_a_training_step_writes_rollout_train_and_time_channels():
    w = RecordingWriter()
    stats = metrics.collect_train_batch_stats(_batch())
    stats["skipped_long"] = 2
    metrics.record_training_stats(w, stats, 7, {"loss": 0.5, "lr": 1e-6, "note": "text", "flag": True}, _batch(),
                                  timings={"rollout": 1.5, "train": 2.5, "other": 9.0})
    s = w.scalars
    assert s["rollout/rewards_mean"] == (0.5, 7) and s["rollout/rewards_max"][0] == 1.0 and s["rollout/accuracy"][0] == 0.5
    assert s["rollout/advantages_mean"][0] == 0.0 and s["rollout/advantages_std"][0] == 1.0
    assert s["rollout/logprobs_mean"][0] == pytest.approx(-1.125)
    assert s["rollout/seq_len_mean"][0] == 3.5 and s["rollout/prompt_len_mean"][0] == 1.5
    assert s["rollout/num_sequences"][0] == 2 and s["rollout/skipped_long"][0] == 2
    assert s["train/loss"][0] == 0.5 and s["train/lr"][0] == 1e-6 and "train/note" not in s
    assert s["time/rollout"][0] == 1.5 and s["time/train"][0] == 2.5 and "time/other" not in s and "time/reward" not in s
    assert w.flushed == 1


def test_empty_batches_write_only_what_they_know():
    w = RecordingWriter()
    metrics.record_training_stats(w, metrics.init_rollout_stats(), 0, None, [])
    assert set(w.scalars) == {"rollout/num_sequences", "rollout/skipped_long", "rollout/total_skipped_long"}


def test_recorder_closes_once(monkeypatch, tmp_path):
    w = RecordingWriter()
    monkeypatch.setattr(metrics, "create_tensorboard_writer", lambda log_dir: w)
    with metrics.MetricsRecorder(str(tmp_path)) as rec:
        rec.record_train_step(step=1, train_result={"loss": 1.0}, train_batch=_batch(), timings={"train": 0.1})
        rec.close()
    rec.close()
    rec.__del__()
    assert w.closed == 1 and w.scalars["train/loss"] == (1.0, 1)
