"""``--tune-params``: pick rollout concurrency and train micro-batch size by measuring memory.

Two stages, both probing from the largest candidate downwards and accepting the first one whose
measured peak memory fraction stays at or under ``mem_frac``:

* rollout: powers of two of ``max_running_prompts`` up to ``--tune-max-samples`` (skipped when the
  user set ``--max-running-prompts``).  A probe allocates the paged KV cache for that many slots at
  the full context length and captures the decode graphs.
* train: the batch is derived from the rollout concurrency (``floor_pow2(rows // n_samples)``
  prompts) and only ``mini_bs`` in {16, 8, 4, 2, 1} is searched; a probe trains one step on
  synthetic full-length rows with random-initialised weights.

Out-of-memory and tensor-parallel divisibility errors mark a candidate as rejected; any other error
propagates.  Same search as ``areno/cli/auto_tune.py:57-330`` in the reference; the probes go through
``Trainer.probe_rollout_cache`` / ``Trainer.train`` of this package.
"""

from __future__ import annotations

import copy
import logging
from collections.abc import Callable
from contextlib import suppress
from dataclasses import dataclass, replace

from ..api.trainer_config import RolloutTrainerConfig, TrainerConfig

logger = logging.getLogger(__name__)
MINI_BS_LADDER = (1, 2, 4, 8, 16)


@dataclass(frozen=True)
class AutoTuneCandidate:
    tp_size: int
    batch_size: int
    n_samples: int
    mini_bs: int
    max_running_prompts: int
    adam_8bit: bool
    keep_rollout_state: bool

    @property
    def train_rows(self) -> int:
        return self.batch_size * self.n_samples

    def describe(self) -> str:
        return (f"tp_size={self.tp_size} batch_size={self.batch_size} n_samples={self.n_samples} "
                f"mini_bs={self.mini_bs} max_running_prompts={self.max_running_prompts} "
                f"adam_8bit={self.adam_8bit} keep_rollout_state={self.keep_rollout_state}")


@dataclass(frozen=True)
class AutoTuneMeasurement:
    candidate: AutoTuneCandidate
    peak_mem_frac: float
    ok: bool
    error: str | None = None

    def describe(self) -> str:
        tail = f" error={self.error}" if self.error else ""
        return f"{self.candidate.describe()} ok={self.ok} peak_mem_frac={self.peak_mem_frac:.4f}{tail}"


@dataclass(frozen=True)
class AutoTuneResult:
    config: TrainerConfig
    measurement: AutoTuneMeasurement | None
    measurements: tuple[AutoTuneMeasurement, ...]


ProbeFn = Callable[[TrainerConfig, AutoTuneCandidate, str], AutoTuneMeasurement]


# ----------------------------------------------------------------------- small helpers
def powers_of_two_up_to(value: int) -> list[int]:
    out, cur = [], 1
    while cur <= value:
        out.append(cur)
        cur <<= 1
    return out or [1]


def floor_power_of_two(value: int) -> int:
    return 1 << (max(int(value), 1).bit_length() - 1)


def sparse_select(items: list, limit: int) -> list:
    """At most ``limit`` items, evenly spread by index, always keeping both ends."""
    if len(items) <= limit:
        return items
    if limit <= 1:
        return [items[-1]]
    last = len(items) - 1
    picks = sorted({round(i * last / (limit - 1)) for i in range(limit)})
    return [items[i] for i in picks]


def mini_bs_values(max_mini_bs: int, rows: int) -> list[int]:
    cap = min(max_mini_bs, rows)
    return [v for v in MINI_BS_LADDER if v <= cap] or [1]


def is_oom_error(message: str) -> bool:
    m = message.lower()
    if "out of memory" in m:
        return True
    if "worker exited without reporting result" in m and (
            "exitcode -9" in m or "during op.train" in m or "during op.probe_rollout_cache" in m):
        return True
    return "failed during op.probe_rollout_cache" in m and any(
        k in m for k in ("nccl", "device error", "external library call failed", "system call"))


def is_tp_compat_error(message: str) -> bool:
    m = message.lower()
    return "tp_size" in m or "divisible by tp" in m or ("divisible" in m and ("head" in m or "kv" in m))


# -------------------------------------------------------------------------- candidates
def _base_candidate(config: RolloutTrainerConfig) -> AutoTuneCandidate:
    return AutoTuneCandidate(tp_size=int(config.tp_size), batch_size=floor_power_of_two(config.batch_size),
                             n_samples=max(int(config.n_samples), 1), mini_bs=1, max_running_prompts=1,
                             adam_8bit=bool(config.adam_8bit), keep_rollout_state=False)


def rollout_candidates(config: RolloutTrainerConfig, *, auto_max_samples: int = 256) -> list[AutoTuneCandidate]:
    """Largest first; at most 16."""
    base = _base_candidate(config)
    rows = max(base.train_rows, 1)
    items = [replace(base, mini_bs=min(base.mini_bs, rows), max_running_prompts=n)
             for n in powers_of_two_up_to(max(int(auto_max_samples), 1))]
    return list(reversed(sparse_select(items, 16)))


def train_template(config: RolloutTrainerConfig, rollout: AutoTuneCandidate, *, auto_max_samples: int) -> AutoTuneCandidate:
    n_samples = max(int(config.n_samples), 1)
    max_rows = max(1, min(int(auto_max_samples), int(rollout.max_running_prompts)))
    batch = max(1, floor_power_of_two(max_rows // n_samples))
    return replace(rollout, batch_size=batch, n_samples=n_samples,
                   mini_bs=min(max(int(config.mini_bs), 1), batch * n_samples), keep_rollout_state=False)


def train_candidates(config: RolloutTrainerConfig, template: AutoTuneCandidate, *, auto_max_samples: int = 256):
    n_samples = max(int(config.n_samples), 1)
    max_batch = max(1, min(int(config.batch_size), max(int(auto_max_samples), 1) // n_samples))
    items = [replace(template, batch_size=b, n_samples=n_samples, mini_bs=m, keep_rollout_state=False)
             for b in powers_of_two_up_to(max_batch) for m in mini_bs_values(max(int(config.mini_bs), 1), b * n_samples)]
    items = sorted(set(items), key=lambda c: (c.train_rows, c.mini_bs))
    return sparse_select(items, 32)


def enumerate_candidates(config: RolloutTrainerConfig, *, auto_max_samples: int = 256) -> list[AutoTuneCandidate]:
    """Every point the tuner may visit, for inspection."""
    ro = rollout_candidates(config, auto_max_samples=auto_max_samples)
    tr = [c for t in ro for c in train_candidates(config, t, auto_max_samples=auto_max_samples)]
    uniq = {c: None for c in [*ro, *tr]}
    return sorted(uniq, key=lambda c: (c.tp_size, c.max_running_prompts, c.train_rows, c.mini_bs))


def enumerate_candidate_groups(config: RolloutTrainerConfig, *, auto_max_samples: int = 256):
    return [rollout_candidates(config, auto_max_samples=auto_max_samples)]


# ------------------------------------------------------------------------------ search
def _first_fit(config, candidates, *, mem_frac: float, probe: ProbeFn, stage: str):
    seen: list[AutoTuneMeasurement] = []
    for i, cand in enumerate(candidates, start=1):
        logger.info("auto tune %s probe %d/%d %s", stage, i, len(candidates), cand.describe())
        m = probe(config, cand, stage)
        seen.append(m)
        logger.info("auto tune %s result %s", stage, m.describe())
        if m.ok and m.peak_mem_frac <= mem_frac:
            return m, seen
    first = seen[0].error if seen else "no candidates"
    raise RuntimeError(f"auto tune {stage} stage could not find a candidate under mem_frac={mem_frac}; "
                       f"first error: {first}")


def auto_tune_config(config: TrainerConfig, *, mem_frac: float = 0.9, auto_max_samples: int = 256,
                     probe_fn: ProbeFn | None = None) -> AutoTuneResult:
    if not 0 < float(mem_frac) <= 1:
        raise ValueError("--mem-frac must be in (0, 1]")
    if int(auto_max_samples) < 1:
        raise ValueError("--tune-max-samples must be >= 1")
    if not isinstance(config, RolloutTrainerConfig):
        raise ValueError("--tune-params currently tunes rollout-based trainers only")
    probe = probe_fn or probe_candidate_with_dummy_run
    measurements: list[AutoTuneMeasurement] = []
    if config.max_running_prompts is not None:
        chosen_rollout = replace(_base_candidate(config), max_running_prompts=int(config.max_running_prompts))
        logger.info("auto tune rollout skipped user_max_running_prompts=%d", config.max_running_prompts)
    else:
        m, seen = _first_fit(config, rollout_candidates(config, auto_max_samples=auto_max_samples),
                             mem_frac=mem_frac, probe=probe, stage="rollout")
        measurements += seen
        chosen_rollout = m.candidate
    template = train_template(config, chosen_rollout, auto_max_samples=auto_max_samples)
    ladder = [replace(template, mini_bs=v)
              for v in reversed(mini_bs_values(max(int(config.mini_bs), 1), template.train_rows))]
    best, seen = _first_fit(config, ladder, mem_frac=mem_frac, probe=probe, stage="train")
    measurements += seen
    c = best.candidate
    tuned = replace(config, tp_size=c.tp_size, batch_size=c.batch_size, n_samples=c.n_samples, mini_bs=c.mini_bs,
                    max_running_prompts=c.max_running_prompts, keep_rollout_state=c.keep_rollout_state)
    logger.info("auto tune selected %s", best.describe())
    return AutoTuneResult(config=tuned, measurement=best, measurements=tuple(measurements))


def format_auto_tune_summary(result: AutoTuneResult) -> str | None:
    import click

    m = result.measurement
    if m is None:
        return None
    c = m.candidate
    return (click.style("AReno-B200 parameter tune selected", fg="bright_green", bold=True)
            + f": tp_size={c.tp_size}, batch_size={c.batch_size}, n_samples={c.n_samples}, mini_bs={c.mini_bs}, "
              f"max_running_prompts={c.max_running_prompts}, adam_8bit={c.adam_8bit}, "
              f"drop_rollout_state={not c.keep_rollout_state}, peak_mem_frac={m.peak_mem_frac:.4f}")


# ------------------------------------------------------------------------------ probes
def dummy_token_budgets(*, max_prompt_tokens: int, max_new_tokens: int, max_context_len: int | None) -> tuple[int, int]:
    prompt = max(int(max_prompt_tokens), 1)
    new = max(int(max_new_tokens), 1)
    if max_context_len is not None and prompt + new > max_context_len:
        prompt = max(1, min(prompt, max_context_len - 1))
        new = max(1, max_context_len - prompt)
    return prompt, new


def _filler_tokens(tokenizer, width: int, text: str) -> list[int]:
    ids = []
    with suppress(Exception):
        ids = list(tokenizer.encode(text, add_special_tokens=False))
    ids = [int(t) for t in ids] or [1]
    reps = (width + len(ids) - 1) // len(ids)
    return (ids * reps)[:width]


def dummy_train_rows(*, prompt_tokens: list[int], response_tokens: list[int], eos_token_id: int, target_rows: int):
    from ..api.models import TrainSequence

    tokens = list(prompt_tokens) + list(response_tokens)
    n_p, n_r = len(prompt_tokens), len(response_tokens)
    row = dict(tokens=tokens, prompt_mask=[True] * n_p + [False] * n_r, loss_mask=[False] * n_p + [True] * n_r,
               logprobs=[0.0] * len(tokens), advantages=[0.0] * n_p + [1.0] * n_r, reward=1.0, eos_token_id=eos_token_id)
    return [TrainSequence(**row) for _ in range(max(int(target_rows), 1))]


def dummy_policy_loss(pack: dict, logprobs):
    """Minimal differentiable loss for memory probing: masked mean negative log-probability."""
    from ..api.loss_fns.layout import masked_mean, response_layout

    loss = -masked_mean(logprobs, response_layout(pack, logprobs))
    return loss, {"loss": loss.detach()}


def probe_candidate_with_dummy_run(config: TrainerConfig, candidate: AutoTuneCandidate, stage: str) -> AutoTuneMeasurement:
    try:
        peak = _run_dummy_probe(config, candidate, stage=stage)
        return AutoTuneMeasurement(candidate, peak, ok=True)
    except (RuntimeError, ValueError) as exc:
        msg = str(exc)
        if is_oom_error(msg) or is_tp_compat_error(msg):
            return AutoTuneMeasurement(candidate, 1.0, ok=False, error=msg)
        raise


def _run_dummy_probe(config: TrainerConfig, candidate: AutoTuneCandidate, *, stage: str) -> float:
    import torch

    from .. import api

    pc = copy.deepcopy(config)
    for name in ("batch_size", "n_samples", "mini_bs", "max_running_prompts", "tp_size", "adam_8bit", "keep_rollout_state"):
        setattr(pc, name, getattr(candidate, name))
    custom = pc.areno_config()
    custom.dummy_load = True
    custom.max_running_prompts = candidate.max_running_prompts
    n_dev = torch.cuda.device_count() if torch.cuda.is_available() else 0
    devices = list(range(min(pc.world_size, n_dev)))
    if devices:
        custom.devices = devices
    trainer = api.Trainer(pc.world_size, pc.ckpt, backend_type=api.Areno, custom_config=custom, metrics_log_dir=None)
    for d in devices:
        torch.cuda.reset_peak_memory_stats(d)
    try:
        trainer.init()
        tok = trainer.get_tokenizer()
        p_len, r_len = dummy_token_budgets(max_prompt_tokens=pc.max_prompt_tokens, max_new_tokens=pc.max_new_tokens,
                                           max_context_len=pc.max_context_len)
        prompt = _filler_tokens(tok, p_len, "Solve the problem step by step. ")
        response = _filler_tokens(tok, r_len, "The answer follows from the previous line. ")
        kw = dict(max_new_tokens=len(response), max_running_prompts=candidate.max_running_prompts,
                  max_prompt_len=len(prompt))
        if stage == "rollout":
            return float(trainer.probe_rollout_cache(**kw))
        trainer.begin_rollout_session()
        try:
            trainer.probe_rollout_cache(**kw)
        finally:
            with suppress(Exception):
                trainer.end_rollout_session()
        eos = int(getattr(tok, "eos_token_id", None) or 0)
        rows = dummy_train_rows(prompt_tokens=prompt, response_tokens=response, eos_token_id=eos,
                                target_rows=candidate.train_rows)
        stats = trainer.train(rows, dummy_policy_loss, mini_bs=candidate.mini_bs)
        worker_peak = float(stats.get("auto_tune_worker_peak_mem_frac", 0.0)) if isinstance(stats, dict) else 0.0
        if worker_peak > 0.0:
            return worker_peak
        peak = 0.0
        for d in devices:
            torch.cuda.synchronize(d)
            total = torch.cuda.get_device_properties(d).total_memory
            peak = max(peak, torch.cuda.max_memory_allocated(d) / total)
        return peak
    finally:
        with suppress(Exception):
            trainer.close()
        if devices:
            torch.cuda.empty_cache()
