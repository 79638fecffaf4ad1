"""Actor training: packing, micro-batch forward/backward, sharded optimizer step.

``pack_train_data`` turns right-padded rollout rows ``(B, T)`` into one packed variable-length
batch plus flat per-action views (an "action" is a position that predicts the next token, i.e.
every token of a row but its last).  Key names and semantics are those of the reference
(``areno/engine/runtime/train_step.py:89-192``) so loss functions written for it run unchanged;
the index construction is a C++ pass instead of a per-row Python loop with ``.item()`` syncs.

``TrainingManager.train`` is the counterpart of ``areno/engine/training.py:31-136``: per pack
forward -> selected log-probs -> ``loss_fn(pack, logprobs)`` -> backward with fp32 main-grad
accumulation; on the last pack of an accumulation group the sharded optimizer reduces, clips,
updates and re-gathers.
"""

from __future__ import annotations

import os
from typing import Any, Callable

import numpy as np
import torch

from ..models.dense import TrainMeta
from ..ops.attention import build_varlen_meta
from ..parallel.context import get_context
from ..utils.log import get_logger
from ..utils.tracing import trace_range
from . import _runtime
from .config import EngineConfig
from .logprobs import lm_head_logprobs
from .optim import ShardedAdamW, lr_for_step

logger = get_logger()

_PER_TOKEN_KEYS = ("advantages", "logprobs", "ref_logprobs", "values", "returns")


def pack_train_data(data_pack: dict[str, Any]) -> dict[str, Any]:
    """Padded rows -> packed varlen batch (CPU tensors in, CPU tensors out)."""
    lengths = data_pack.get("lengths")
    input_ids = data_pack.get("input_ids")
    if not isinstance(lengths, torch.Tensor) or not isinstance(input_ids, torch.Tensor):
        return data_pack
    if input_ids.ndim != 2 or lengths.ndim != 1 or lengths.numel() != input_ids.shape[0]:
        return data_pack
    prompt_mask = data_pack.get("prompt_mask")
    advantages = data_pack.get("advantages")
    rollout_logprobs = data_pack.get("logprobs")
    if not all(isinstance(x, torch.Tensor) for x in (prompt_mask, advantages, rollout_logprobs)):
        return data_pack
    batch, width = input_ids.shape
    len_np = np.clip(lengths.detach().cpu().numpy().astype(np.int64), 1, width)
    rows, cols, aidx, arows = _runtime.pack_indices(len_np, width)
    rows_t, cols_t = torch.from_numpy(rows), torch.from_numpy(cols)
    aidx_t, arows_t = torch.from_numpy(aidx), torch.from_numpy(arows)
    ids_cpu = input_ids.detach().cpu()
    packed_ids = ids_cpu[rows_t, cols_t]
    # per-action signals are read at the *target* token (column + 1 of the action site)
    a_rows, a_cols = arows_t, cols_t[aidx_t] + 1
    response_mask = ~prompt_mask.detach().cpu()[a_rows, a_cols].to(torch.bool)
    loss_mask = data_pack.get("loss_mask")
    if isinstance(loss_mask, torch.Tensor):
        response_mask = response_mask & loss_mask.detach().cpu()[a_rows, a_cols].to(torch.bool)
    cu = np.zeros(batch + 1, dtype=np.int32)
    np.cumsum(len_np, out=cu[1:])
    packed = dict(data_pack)
    packed.update({
        "input_ids": packed_ids.unsqueeze(0),
        "position_ids": cols_t.unsqueeze(0),
        "train_cu_seqlens": torch.from_numpy(cu),
        "train_max_seqlen": int(len_np.max()),
        "packed_response_mask": response_mask,
        "packed_advantages": advantages.detach().cpu()[a_rows, a_cols].float(),
        "packed_logprobs": rollout_logprobs.detach().cpu()[a_rows, a_cols].float(),
        "packed_seq_ids": arows_t,
        "packed_num_sequences": batch,
        "_action_index": aidx_t,
        "_seq_lengths": [int(x) for x in len_np],
    })
    for key in ("ref_logprobs", "values", "returns"):        # each optional signal on its own
        extra = data_pack.get(key)
        if isinstance(extra, torch.Tensor):
            packed["packed_" + key] = extra.detach().cpu()[a_rows, a_cols].float()
    return packed


def to_device(pack: Any, device: torch.device) -> Any:
    """Move every tensor of a pack to ``device`` (pinned staging + async copy on CUDA).  Dicts, lists and tuples are
    walked recursively and rebuilt; anything else is passed through unchanged (``areno/engine/data.py``)."""
    device = torch.device(device)
    if isinstance(pack, torch.Tensor):
        if pack.device == device:
            return pack
        if device.type == "cuda" and pack.device.type == "cpu" and not pack.is_pinned() and pack.numel() > 0:
            pack = pack.pin_memory()
        return pack.to(device, non_blocking=True)
    if isinstance(pack, dict):
        return {k: to_device(v, device) for k, v in pack.items()}
    if isinstance(pack, tuple) and hasattr(pack, "_fields"):          # named tuple: positional constructor
        return type(pack)(*(to_device(v, device) for v in pack))
    if isinstance(pack, (list, tuple)):
        return type(pack)(to_device(v, device) for v in pack)
    return pack


def split_data_pack_by_dp(pack: dict[str, Any], dp_size: int) -> list[dict[str, Any]]:
    """Strided ``rank::dp`` split of every batch-major tensor; a batch smaller than ``dp_size`` is
    replicated (``areno/engine/runtime/common.py:76-109``)."""
    ids = pack.get("input_ids")
    if dp_size <= 1 or not isinstance(ids, torch.Tensor):
        return [pack for _ in range(max(dp_size, 1))]
    batch = ids.shape[0]
    if batch < dp_size:
        return [pack for _ in range(dp_size)]
    shards = []
    for r in range(dp_size):
        shard = {}
        for k, v in pack.items():
            if isinstance(v, torch.Tensor) and v.ndim >= 1 and v.shape[0] == batch:
                shard[k] = v[r::dp_size]
            elif isinstance(v, list) and len(v) == batch:
                shard[k] = v[r::dp_size]
            else:
                shard[k] = v
        shards.append(shard)
    return shards


def balanced_partition(lengths: list[int], parts: int) -> list[list[int]]:
    """Deal sequences out to ``parts`` data-parallel ranks so that every rank gets the same number of sequences
    (within one) and nearly the same number of tokens: longest first, each to the rank with the fewest tokens among
    those that still have room.  Returns the indices per rank; deterministic, so every rank computes the same plan.

    The reference deals rows out by stride (``areno/engine/runtime/common.py:76-109``), which balances counts but
    not tokens; the slowest rank then sets the step time."""
    n = len(lengths)
    quota = [n // parts + (1 if r < n % parts else 0) for r in range(parts)]
    load = [0] * parts
    out: list[list[int]] = [[] for _ in range(parts)]
    for i in sorted(range(n), key=lambda j: (-lengths[j], j)):
        r = min((r for r in range(parts) if len(out[r]) < quota[r]), key=lambda r: (load[r], r))
        out[r].append(i)
        load[r] += lengths[i]
    return [sorted(ix) for ix in out]


def pack_into_bins(lengths: list[int], token_cap: int, n_bins: int | None = None) -> list[list[int]]:
    """Group sequences into micro-batches of at most ``token_cap`` tokens (a single longer sequence gets a bin of
    its own).  With ``n_bins`` the result has exactly that many bins when they can hold the tokens (longest first
    into the emptiest bin that still has room), so that all data-parallel ranks run the same number of micro-batches;
    otherwise bins are filled first-fit in decreasing order of length."""
    order = sorted(range(len(lengths)), key=lambda j: (-lengths[j], j))
    if n_bins is None:
        bins: list[list[int]] = []
        fill: list[int] = []
        for i in order:
            for b in range(len(bins)):
                if fill[b] + lengths[i] <= token_cap:
                    bins[b].append(i)
                    fill[b] += lengths[i]
                    break
            else:
                bins.append([i])
                fill.append(lengths[i])
        return [sorted(b) for b in bins]
    bins = [[] for _ in range(n_bins)]
    fill = [0] * n_bins
    for i in order:
        fits = [b for b in range(n_bins) if fill[b] + lengths[i] <= token_cap]
        b = min(fits or range(n_bins), key=lambda b: (fill[b], b))
        bins[b].append(i)
        fill[b] += lengths[i]
    return [sorted(b) for b in bins if b]


class TrainStats(dict):
    """Statistics of one training micro-step (``loss``, ``stepped``, ``global_step``, ``metrics``, ``num_tokens``): a
    dict whose entries also read as attributes, the form of the reference's dataclass
    (``areno/engine/data/batch.py:19-24``), so ``stats.loss`` and ``stats["loss"]`` both work."""

    def __getattr__(self, name: str):
        try:
            return self[name]
        except KeyError:
            raise AttributeError(name) from None


def merge_train_stats(stats: list[dict]) -> dict:
    """Mean over DP ranks of scalar stats (``areno/engine/runtime/common.py:112-132``)."""
    stats = [s for s in stats if s]
    if not stats:
        return TrainStats()
    out = TrainStats(stats[0])
    out["loss"] = sum(s["loss"] for s in stats) / len(stats)
    metrics: dict[str, float] = {}
    for key in stats[0].get("metrics", {}):
        vals = [s["metrics"][key] for s in stats if key in s.get("metrics", {})]
        if vals and all(isinstance(v, (int, float)) for v in vals):
            metrics[key] = sum(vals) / len(vals)
        elif vals:
            metrics[key] = vals[0]
    out["metrics"] = metrics
    return out


class TrainingManager:
    def __init__(self, model, config: EngineConfig, device, loss_fn: Callable | None = None):
        self.model = model
        self.config = config
        self.device = torch.device(device)
        self.loss_fn = loss_fn
        ctx = get_context()
        want_sp = config.runtime.sequence_parallel or os.environ.get("ARENO_SEQUENCE_PARALLEL", "0") == "1"
        self.sequence_parallel = bool(want_sp and ctx.tp_size > 1 and getattr(model, "supports_sequence_parallel", False))
        self.optimizer = ShardedAdamW(model, config.optimizer, sequence_parallel=self.sequence_parallel)
        self.global_step = 0
        self.grad_clip_norm = config.optimizer.grad_clip_norm

    # ------------------------------------------------------------------ public
    def train(self, packs: list, gradient_accumulation_steps: int | None = None) -> list[dict]:
        """``packs``: list of micro-batches, each a list of per-DP-rank shards (or a single pack)."""
        n = len(packs)
        ctx = get_context()
        if ctx.ep_size > 1 and ctx.ep_runtime is not None:
            # every micro-batch is a group-wide token exchange: a rank with fewer of them would leave the others
            # waiting inside one.  All ranks learn the spread here and fail together instead.
            most, neg_least = ctx.ep_runtime.agree_max([n, -n])
            if most != -neg_least:
                raise ValueError(f"expert parallelism needs the same number of micro-batches on every rank; this call "
                                 f"has between {-neg_least} and {most} (this rank: {n})")
        accum = n if not gradient_accumulation_steps else max(1, min(gradient_accumulation_steps, n))
        results = []
        for i, shards in enumerate(packs):
            group_pos = i % accum
            remaining = n - (i - group_pos)
            group = min(accum, remaining)
            allow_step = group_pos == group - 1
            results.append(self.train_step(shards, allow_step=allow_step, grad_scale=group, defer_sync=True))
        out = [_materialize(r) for r in results]
        if self.device.type == "cuda":
            from ..ops import _lib

            _lib.check_status(self.device)   # a kernel that gave up on a bounded wait must fail the step, not pass silently
        return out

    def forward_logprobs(self, pack: dict, need_entropy: bool = False):
        """Packed forward to per-action log-probs ``[num_actions]`` (fp32)."""
        ids = pack["input_ids"].reshape(-1)
        pos = pack["position_ids"].reshape(-1)
        lens = pack.get("_seq_lengths")
        if lens is None:
            cu = pack["train_cu_seqlens"].tolist()
            lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
        meta = TrainMeta(build_varlen_meta(lens, device=self.device),
                         activation_checkpointing=self.config.runtime.activation_checkpointing,
                         checkpoint_layers=self._checkpoint_layers(int(ids.numel())),
                         layer_grad_hook=getattr(self, "_layer_grad_hook", None),
                         sequence_parallel=self.sequence_parallel)
        out = self.model(ids, pos, meta)
        aidx = pack["_action_index"]
        hidden = out.hidden_states.index_select(0, aidx)
        targets = ids.index_select(0, aidx + 1)
        return lm_head_logprobs(self.model.lm_head, hidden, targets, self.config.runtime.logprob_chunk,
                                need_entropy=need_entropy, softcap=self.model.cfg.final_logit_softcapping)

    def _checkpoint_layers(self, tokens: int) -> int | None:
        """How many layers to recompute in backward.  Checkpointing exists to save memory; when the
        device has room, layers keep their activations and skip the recompute.  Decided from the
        free memory seen once the optimizer state exists, with a fixed reserve for transients."""
        if not self.config.runtime.activation_checkpointing or self.device.type != "cuda":
            return None
        mc = self.model.cfg
        n_layers = mc.num_hidden_layers
        cached = getattr(self, "_ckpt_cache", None)
        ctx = get_context()
        if cached is not None and (cached[0] >= tokens or ctx.ep_size > 1):
            return cached[1]      # expert parallel: decided once for all ranks (see below)
        self.optimizer._ensure_state()
        if ctx.ep_size > 1:
            tokens = ctx.ep_runtime.agree_max([tokens])[0]
        tp = max(1, ctx.tp_size)
        qkv_w = (mc.num_attention_heads + 2 * mc.num_key_value_heads) * mc.head_dim // tp
        inter = (mc.moe_intermediate_size * max(1, mc.num_experts_per_tok) if mc.num_experts else mc.intermediate_size)
        per_token = 2 * (5 * mc.hidden_size + qkv_w + mc.num_attention_heads * mc.head_dim // tp + 3 * inter // tp)
        per_layer = per_token * max(tokens, 1)
        free, _total = torch.cuda.mem_get_info(self.device)
        free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        reserve = int(float(os.environ.get("ARENO_CKPT_RESERVE_GB", "26")) * (1 << 30))
        keep = max(0, int((free - reserve) // max(per_layer, 1)))
        n_ckpt = max(0, n_layers - keep)
        if ctx.ep_size > 1:
            # a recomputed layer repeats its token exchange in backward: every rank must recompute the same layers.
            # The first micro-batch of a run reaches this point on every rank, later ones use the cached answer.
            n_ckpt = ctx.ep_runtime.agree_max([n_ckpt])[0]
        self._ckpt_cache = (tokens, n_ckpt)
        logger.info("activation checkpointing: recompute %d of %d layers (free=%.1f GB, per-layer=%.2f GB)", n_ckpt,
                    n_layers, free / 2**30, per_layer / 2**30)
        return n_ckpt

    def train_step(self, shards, *, allow_step: bool, grad_scale: int, defer_sync: bool = False) -> dict:
        ctx = get_context()
        self.model.train()
        pack = shards[ctx.dp_rank] if isinstance(shards, (list, tuple)) else shards
        pack = pack_train_data(pack)
        loss_fn = pack.get("_loss_fn") or self.loss_fn
        if loss_fn is None:
            raise ValueError("no loss function: pass loss_fn or stamp '_loss_fn' on the pack")
        with trace_range("train/h2d"):
            pack = to_device(pack, self.device)
        # last micro-batch of the window: gradient buckets are handed to the reduce-scatter as backward passes them
        self._layer_grad_hook = self.optimizer.begin_overlap() if allow_step and hasattr(self.optimizer, "begin_overlap") \
            else None
        # Expert parallelism: the ranks' micro-batches differ in size, but every MoE call of this forward, of a
        # recomputed forward and of the backward must use the communicator of one common size
        ep_rt = ctx.ep_runtime if ctx.ep_size > 1 else None
        pin = ep_rt.pinned(ep_rt.agree_max([int(pack["input_ids"].numel())])[0]) if ep_rt is not None else None
        if pin is not None:
            pin.__enter__()
        try:
            with trace_range("train/forward"):
                logprobs = self.forward_logprobs(pack)
            self._layer_grad_hook = None
            with trace_range("train/loss"):
                loss_out = loss_fn(pack, logprobs)
            metrics = None
            if isinstance(loss_out, tuple):
                loss, metrics = loss_out
            else:
                loss = loss_out
            if not isinstance(loss, torch.Tensor):
                raise TypeError("train_loss_fn must return a torch.Tensor")
            with trace_range("train/backward"):
                (loss / max(grad_scale, 1)).backward()
        finally:
            if pin is not None:
                pin.__exit__(None, None, None)
        grad_norm = None
        lr = self.optimizer.lr
        if allow_step:
            if hasattr(self.model, "finalize_router_expert_bias"):
                self.model.finalize_router_expert_bias(ctx.tp_group, ctx.dp_group)
            lr = lr_for_step(self.config.optimizer, self.global_step + 1)
            self.optimizer.lr = lr
            with trace_range("train/optimizer_step"):
                grad_norm = self.optimizer.step(lr=lr, clip_norm=self.grad_clip_norm)
            self.global_step += 1
        else:
            with trace_range("train/fold_grads"):
                self.optimizer.fold_param_grads()
        out_metrics = dict(metrics) if metrics else {}
        out_metrics["lr"] = lr
        if grad_norm is not None:
            out_metrics["grad_norm"] = grad_norm
        result = {
            "loss": loss.detach(),
            "stepped": allow_step,
            "global_step": self.global_step,
            "metrics": out_metrics,
            "num_tokens": int(pack["input_ids"].numel()),
        }
        # device scalars are read back once per call to train(), not once per micro-batch
        return result if defer_sync else _materialize(result)


def _scalar(v):
    if isinstance(v, torch.Tensor):
        return float(v.detach().float().reshape(-1)[0].cpu()) if v.numel() else 0.0
    return v


def _materialize(result: dict) -> dict:
    out = dict(result)
    out["loss"] = _scalar(result["loss"])
    out["metrics"] = {k: _scalar(v) for k, v in result.get("metrics", {}).items()}
    return out
