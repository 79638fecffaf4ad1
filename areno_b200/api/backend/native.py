"""Native backend: maps the SDK's ``Backend`` calls onto ``areno_b200.engine.ArenoEngine``.

Behaviour kept from the reference adapter (``areno/api/backend/areno/backend.py:39-588``): public
sampling parameters are translated to engine ones (greedy => temperature 0; pad / bos / unk and -
unless ``ignore_eos`` - every special id except EOS and stop ids are suppressed), prompts are
replicated ``n_samples`` times in a flat list, train sequences are right-padded into packs with
the caller's loss function stamped on each pack, SFT gets global-token-mean annotations, and
per-pack metrics are averaged (rollout-policy diagnostics from the first micro-batch only).
"""

from __future__ import annotations

import itertools
import time
from typing import Any, Callable

import numpy as np
import torch

from ..config import ArenoConfig
from ..context import Context
from ..loss_fns import sft_loss_fn
from ..models import BackendType, RolloutResult, RolloutSequence, SamplingParams, TrainSequence
from ..roles import ModelRole
from .base import Backend, register_backend


def explicit_suppress_token_ids(tokenizer) -> tuple[int, ...]:
    out = []
    for attr in ("pad_token_id", "bos_token_id", "unk_token_id"):
        v = getattr(tokenizer, attr, None)
        if isinstance(v, int) and not isinstance(v, bool):
            out.append(v)
    return tuple(dict.fromkeys(out))


def rollout_options(ctx: Context, sampling_params: SamplingParams) -> dict:
    from ...engine.inference import SamplingParams as EngineSamplingParams

    eos = () if sampling_params.ignore_eos else tuple(ctx.eos_token_ids)
    stop = tuple(sampling_params.stop_token_ids or ())
    suppress = set(explicit_suppress_token_ids(ctx.tokenizer)) if ctx.tokenizer is not None else set()
    if not sampling_params.ignore_eos and ctx.tokenizer is not None:
        suppress.update(int(t) for t in (getattr(ctx.tokenizer, "all_special_ids", ()) or ()))
    suppress_ids = tuple(sorted(t for t in suppress if t not in {*eos, *stop}))
    cfg = ctx.custom_config or ArenoConfig()
    if not isinstance(cfg, ArenoConfig):
        raise TypeError(f"native backend requires ArenoConfig, got {type(cfg)!r}")
    return {
        "max_prompt_len": sampling_params.max_prompt_len,
        "eos_token_id": eos,
        "max_running_prompts": cfg.max_running_prompts,
        "decode_progress_interval_s": cfg.decode_progress_interval_s,
        "sampling_params": EngineSamplingParams(
            temperature=0.0 if sampling_params.greedy else sampling_params.temperature, top_p=sampling_params.top_p,
            top_k=max(0, sampling_params.top_k), stop_token_ids=stop, suppress_token_ids=suppress_ids,
            min_new_tokens=max(0, int(getattr(sampling_params, "min_new_tokens", 0) or 0)),
            seed=getattr(sampling_params, "seed", None)),
    }


_NP_DTYPES = {torch.long: np.int64, torch.int32: np.int32, torch.bool: np.bool_, torch.float32: np.float32}


def pad_rows(rows: list[list], *, dtype, fill_value=0, width: int | None = None) -> torch.Tensor:
    """Right-pad ragged Python lists into one ``(len(rows), width)`` tensor.  The rows are flattened once and
    scattered with index arithmetic (one conversion for the whole batch instead of one per row)."""
    lens = np.fromiter((len(r) for r in rows), dtype=np.int64, count=len(rows))
    width = int(lens.max()) if (width is None and len(rows)) else int(width or 0)
    np_dtype = _NP_DTYPES[dtype]
    out = np.full((len(rows), width), fill_value, dtype=np_dtype)
    take = np.minimum(lens, width)
    total = int(take.sum())
    if total:
        if bool((take == lens).all()):
            flat = np.fromiter(itertools.chain.from_iterable(rows), dtype=np_dtype, count=total)
        else:
            flat = np.fromiter(itertools.chain.from_iterable(r[:width] for r in rows), dtype=np_dtype, count=total)
        row_idx = np.repeat(np.arange(len(rows)), take)
        starts = np.cumsum(take) - take
        col_idx = np.arange(total) - np.repeat(starts, take)
        out[row_idx, col_idx] = flat
    return torch.from_numpy(out)


def make_train_pack(seqs: list[TrainSequence]) -> dict[str, torch.Tensor]:
    """Right-padded ``(B, max_len)`` tensors: ``input_ids`` (padded with EOS), ``labels``, ``lengths``,
    ``prompt_mask`` (True on prompt and padding), ``logprobs``, ``advantages`` and, when any
    sequence carries them, ``loss_mask`` / ``returns`` / ``values`` / ``ref_logprobs``."""
    if not seqs:
        raise ValueError("train batch is empty")
    eos = seqs[0].eos_token_id
    lengths = torch.tensor([len(s.tokens) for s in seqs], dtype=torch.int32)
    width = int(lengths.max())
    ids = pad_rows([s.tokens for s in seqs], dtype=torch.long, fill_value=eos, width=width)
    pack = {
        "input_ids": ids,
        "labels": ids.clone(),
        "lengths": lengths,
        "prompt_mask": pad_rows([s.prompt_mask for s in seqs], dtype=torch.bool, fill_value=True, width=width),
        "logprobs": pad_rows([s.logprobs for s in seqs], dtype=torch.float32, width=width),
        "advantages": pad_rows([s.advantages for s in seqs], dtype=torch.float32, width=width),
    }
    if any(s.loss_mask for s in seqs):
        rows = [s.loss_mask if s.loss_mask else [not m for m in s.prompt_mask] for s in seqs]
        pack["loss_mask"] = pad_rows(rows, dtype=torch.bool, fill_value=False, width=width)
    for key in ("returns", "values", "ref_logprobs"):
        if any(getattr(s, key) for s in seqs):
            pack[key] = pad_rows([getattr(s, key) for s in seqs], dtype=torch.float32, width=width)
    return pack


def _is_sft(loss_fn: Callable) -> bool:
    return loss_fn is sft_loss_fn or getattr(loss_fn, "func", None) is sft_loss_fn


def sft_target_token_count(seqs: list[TrainSequence]) -> int:
    n = 0
    for s in seqs:
        length = min(len(s.tokens), len(s.prompt_mask))
        for i in range(1, length):
            ok = not s.prompt_mask[i]
            if s.loss_mask:
                ok = ok and i < len(s.loss_mask) and s.loss_mask[i]
            n += int(ok)
    return n


def annotate_sft_token_mean_packs(packs, counts, *, gradient_accumulation_steps) -> None:
    if not packs:
        return
    accum = len(packs) if gradient_accumulation_steps is None else max(int(gradient_accumulation_steps), 1)
    for g0 in range(0, len(packs), accum):
        g1 = min(g0 + accum, len(packs))
        total = max(sum(counts[g0:g1]), 1)
        for p in packs[g0:g1]:
            p["_sft_total_target_tokens"] = total
            p["_sft_grad_scale"] = g1 - g0


def _is_rollout_policy_metric(key: str) -> bool:
    return key in {"ratio_mean", "ratio_std", "rollout_logprobs_mean", "train_logprobs_mean"} or key.startswith("logp_diff")


def pad_token_id(ctx: Context) -> int:
    tok = ctx.tokenizer
    t = getattr(tok, "pad_token_id", None)
    if t is None:
        t = getattr(tok, "eos_token_id", None)
    if t is None:
        if ctx.eos_token_ids:
            return int(ctx.eos_token_ids[0])
        raise ValueError("tokenizer must define pad_token_id or eos_token_id")
    return int(t)


@register_backend(BackendType.Areno)
class NativeBackend(Backend):
    def __init__(self, engine=None):
        super().__init__()
        self._engine = engine

    def _require(self):
        if self._engine is None:
            raise RuntimeError("backend is not initialized")
        return self._engine

    def initialize(self, ctx: Context) -> None:
        if self._engine is not None:
            return
        from ...engine import ArenoEngine, OptimizerConfig, RuntimeConfig

        cfg = ctx.custom_config or ArenoConfig()
        if not isinstance(cfg, ArenoConfig):
            raise TypeError(f"native backend requires ArenoConfig, got {type(cfg)!r}")
        world, tp = int(ctx.world_size), int(cfg.tp_size)
        if world % tp != 0:
            raise ValueError(f"world_size={world} must be divisible by tp_size={tp}")
        dp = world // tp if cfg.dp_size is None else int(cfg.dp_size)
        if dp * tp != world:
            raise ValueError(f"dp_size * tp_size must equal world_size, got {dp} * {tp} != {world}")
        devices = cfg.devices if cfg.devices is not None else list(range(world))
        self._engine = ArenoEngine.from_pretrained(
            cfg.model_path or ctx.model_path, tp_size=tp, dp_size=dp, devices=devices, dummy_load=cfg.dummy_load,
            optimizer_config=OptimizerConfig(**cfg.optimizer), runtime_config=RuntimeConfig(**cfg.runtime),
            model_config=cfg.model_config, launcher=cfg.launcher, max_running_seqs=cfg.max_running_prompts,
            seed=cfg.seed, rollout_tp_size=cfg.rollout_tp_size, expert_parallel=cfg.expert_parallel)

    def close(self) -> None:
        engine, self._engine = self._engine, None
        if engine is not None:
            engine.close()

    def dp_size(self, ctx: Context) -> int:
        return int(self._require().config.dp_size)

    def model_context_len(self, ctx: Context) -> int | None:
        return int(self._require().config.model.max_position_embeddings)

    # ----------------------------------------------------------------- rollout
    def begin_rollout_session(self, ctx):
        self._require().begin_rollout_session()

    async def begin_rollout_session_async(self, ctx):
        await self._require().begin_rollout_session_async()

    async def sync_rollout_session_async(self, ctx):
        await self._require().sync_rollout_session_async()

    def end_rollout_session(self, ctx):
        self._require().end_rollout_session()

    async def end_rollout_session_async(self, ctx):
        await self._require().end_rollout_session_async()

    def probe_rollout_cache(self, ctx, *, max_new_tokens, max_running_prompts, max_prompt_len) -> float:
        return self._require().probe_rollout_cache(max_new_tokens=max_new_tokens,
                                                   max_running_prompts=max_running_prompts,
                                                   max_prompt_len=max_prompt_len)

    @staticmethod
    def _to_results(out, n_prompts: int, n_samples: int) -> list[RolloutResult]:
        results = []
        for i in range(n_prompts):
            seqs = []
            for j in range(n_samples):
                k = i * n_samples + j
                seqs.append(RolloutSequence(resp_tokens=list(out.tokens[k]), resp_logprobs=list(out.logprobs[k])))
            results.append(RolloutResult(sequences=seqs))
        return results

    def _flat(self, prompt_tokens, n_samples):
        return [list(p) for p in prompt_tokens for _ in range(n_samples)]

    def rollout_batch(self, ctx, prompt_tokens, n_samples, sampling_params) -> list[RolloutResult]:
        opts = rollout_options(ctx, sampling_params)
        flat = self._flat(prompt_tokens, n_samples)
        out = self._require().generate_rollout(
            flat, max_new_tokens=sampling_params.max_new_tokens, max_running_prompts=opts["max_running_prompts"],
            max_prompt_len=opts["max_prompt_len"], eos_token_id=opts["eos_token_id"],
            sampling_params=opts["sampling_params"], decode_progress_interval_s=opts["decode_progress_interval_s"],
            local=self._local_data(ctx))
        return self._to_results(out, len(prompt_tokens), n_samples)

    @staticmethod
    def _local_data(ctx) -> bool:
        return bool(getattr(ctx.custom_config, "spmd_local_data", False))

    async def rollout_batch_async(self, ctx, prompt_tokens, n_samples, sampling_params) -> list[RolloutResult]:
        opts = rollout_options(ctx, sampling_params)
        flat = self._flat(prompt_tokens, n_samples)
        out = await self._require().generate_rollout_async(
            flat, max_new_tokens=sampling_params.max_new_tokens, max_running_prompts=opts["max_running_prompts"],
            max_prompt_len=opts["max_prompt_len"], eos_token_id=opts["eos_token_id"],
            sampling_params=opts["sampling_params"], decode_progress_interval_s=0.0)
        return self._to_results(out, len(prompt_tokens), n_samples)

    # ------------------------------------------------------------------- train
    def train(self, ctx, batch_data, loss_fn, mini_bs, gradient_accumulation_steps=None) -> dict[str, Any]:
        t0 = time.perf_counter()
        if not batch_data:
            raise ValueError("train batch is empty")
        mini_bs = max(int(mini_bs), 1)
        packs, counts = [], []
        sft = _is_sft(loss_fn)
        for s in range(0, len(batch_data), mini_bs):
            chunk = batch_data[s:s + mini_bs]
            pack = make_train_pack(chunk)
            pack["_loss_fn"] = loss_fn
            packs.append(pack)
            if sft:      # a walk over every token on the host: only the token-mean SFT loss needs the counts
                counts.append(sft_target_token_count(chunk))
        if sft:
            annotate_sft_token_mean_packs(packs, counts, gradient_accumulation_steps=gradient_accumulation_steps)
        stats = self._require().step(packs, gradient_accumulation_steps=gradient_accumulation_steps,
                                     local=self._local_data(ctx))
        return self._reduce_stats(stats, time.perf_counter() - t0)

    @staticmethod
    def _reduce_stats(stats: list[dict], elapsed: float) -> dict[str, Any]:
        if not stats:
            return {}
        out: dict[str, Any] = {"loss": sum(s["loss"] for s in stats) / len(stats)}
        keys: list[str] = []
        for s in stats:
            for k in s.get("metrics", {}):
                if k not in keys:
                    keys.append(k)
        for k in keys:
            vals = [s["metrics"][k] for s in stats if k in s.get("metrics", {})
                    and isinstance(s["metrics"][k], (int, float))]
            if not vals:
                continue
            if _is_rollout_policy_metric(k):
                out[k] = vals[0]          # first micro-batch: measured before any update of this step
            elif k in ("lr", "grad_norm"):
                out[k] = vals[-1]
            else:
                out[k] = sum(vals) / len(vals)
        out["global_step"] = stats[-1].get("global_step", 0)
        out["num_microbatches"] = len(stats)
        out["backend_train_time_s"] = elapsed
        return out

    # ------------------------------------------------------------------- roles
    def ensure_roles(self, ctx, roles: dict[str, ModelRole]) -> None:
        self._require().ensure_roles(roles)

    def score_logprobs(self, ctx, role, token_rows, *, microbatch_size: int = 8):
        return self._require().score_logprobs(role, token_rows, pad_token_id=pad_token_id(ctx),
                                              microbatch_size=microbatch_size)

    def score_values(self, ctx, role, token_rows):
        return self._require().score_values(role, token_rows, pad_token_id=pad_token_id(ctx))

    def score_rewards(self, ctx, role, token_rows):
        return self._require().score_rewards(role, token_rows, pad_token_id=pad_token_id(ctx))

    def train_values(self, ctx, role, batch_data, mini_bs, gradient_accumulation_steps=None, *,
                     cliprange_value: float = 0.5, value_loss_coef: float = 0.5):
        packs = [make_train_pack(batch_data[s:s + mini_bs]) for s in range(0, len(batch_data), mini_bs)]
        return self._require().train_values(role, packs, gradient_accumulation_steps=gradient_accumulation_steps,
                                            cliprange_value=cliprange_value, value_loss_coef=value_loss_coef)

    def save_checkpoint(self, ctx, path: str) -> str:
        return self._require().save_checkpoint(path)
