"""TensorBoard recording of rollout / train / time scalars (``rollout/*``, ``train/*``, ``time/*``
channels as in ``areno/api/metrics.py:16-174`` of the reference)."""

from __future__ import annotations

import numpy as np


class JsonlScalarWriter:
    """Stand-in for ``SummaryWriter`` when no TensorBoard package is installed: one JSON object per scalar
    (``{"tag", "value", "step", "time"}``) appended to ``<log_dir>/metrics.jsonl``."""

    def __init__(self, log_dir: str):
        import os

        os.makedirs(log_dir, exist_ok=True)
        self.path = os.path.join(log_dir, "metrics.jsonl")
        self._fh = open(self.path, "a")

    def add_scalar(self, tag: str, value, step: int) -> None:
        import json
        import time

        self._fh.write(json.dumps({"tag": tag, "value": float(value), "step": int(step), "time": time.time()}) + "\n")

    def flush(self) -> None:
        self._fh.flush()

    def close(self) -> None:
        if not self._fh.closed:
            self._fh.close()


def create_tensorboard_writer(log_dir: str):
    try:
        from torch.utils.tensorboard import SummaryWriter
    except ImportError:
        try:
            from tensorboardX import SummaryWriter
        except ImportError:
            return JsonlScalarWriter(log_dir)
    return SummaryWriter(log_dir=log_dir)


def init_rollout_stats(skipped_long: int = 0, total_skipped_long: int = 0) -> dict:
    return {"rewards": [], "logprobs": [], "advantages": [], "seq_len": [], "prompt_len": [], "response_len": [],
            "skipped_long": skipped_long, "total_skipped_long": total_skipped_long}


def record_rollout_sequence_stats(stats, *, prefix_len: int, response_logprobs, response_len: int) -> None:
    stats["logprobs"].extend(response_logprobs)
    stats["seq_len"].append(prefix_len + response_len)
    stats["prompt_len"].append(prefix_len)
    stats["response_len"].append(response_len)


def collect_train_batch_stats(train_batch) -> dict:
    """Response-side statistics of a list of ``TrainSequence`` (prompt positions are masked out)."""
    stats = init_rollout_stats()
    for seq in train_batch:
        mask = list(seq.prompt_mask)
        resp_lp = [v for v, is_prompt in zip(seq.logprobs, mask) if not is_prompt]
        stats["rewards"].append(seq.reward)
        stats["advantages"].extend(v for v, is_prompt in zip(seq.advantages, mask) if not is_prompt)
        record_rollout_sequence_stats(stats, prefix_len=sum(1 for m in mask if m), response_logprobs=resp_lp,
                                      response_len=len(resp_lp))
    return stats


def record_training_stats(writer, stats, step, train_res, train_batch, timings: dict[str, float] | None = None) -> None:
    rewards = np.asarray(stats.get("rewards", []), dtype=np.float32)
    adv = np.asarray(stats.get("advantages", []), dtype=np.float32)
    lp = np.asarray(stats.get("logprobs", []), dtype=np.float32)
    if rewards.size:
        writer.add_scalar("rollout/rewards_mean", rewards.mean(), step)
        writer.add_scalar("rollout/rewards_std", rewards.std(), step)
        writer.add_scalar("rollout/rewards_max", rewards.max(), step)
        writer.add_scalar("rollout/rewards_min", rewards.min(), step)
        writer.add_scalar("rollout/accuracy", (rewards > 0).mean(), step)
    if adv.size:
        writer.add_scalar("rollout/advantages_mean", adv.mean(), step)
        writer.add_scalar("rollout/advantages_std", adv.std(), step)
    if lp.size:
        writer.add_scalar("rollout/logprobs_mean", lp.mean(), step)
    for key in ("seq_len", "prompt_len", "response_len"):
        if stats.get(key):
            writer.add_scalar(f"rollout/{key}_mean", float(np.mean(stats[key])), step)
    writer.add_scalar("rollout/num_sequences", len(train_batch), step)
    for key in ("skipped_long", "total_skipped_long"):
        if key in stats:
            writer.add_scalar(f"rollout/{key}", stats[key], step)
    for key, value in (train_res or {}).items():
        if isinstance(value, (int, float)):
            writer.add_scalar(f"train/{key}", value, step)
    src = timings or stats
    for key in ("rollout", "reward", "advantage", "train"):
        if key in src:
            writer.add_scalar(f"time/{key}", src[key], step)
    writer.flush()


class MetricsRecorder:
    def __init__(self, log_dir: str):
        self._writer = create_tensorboard_writer(log_dir)
        self._closed = False

    def record_train_step(self, *, step: int, train_result, train_batch, timings: dict[str, float] | None = None):
        record_training_stats(self._writer, collect_train_batch_stats(train_batch), step, train_result, train_batch,
                              timings=timings)

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            self._writer.close()

    def __enter__(self):
        return self

    def __exit__(self, *_exc) -> None:
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
