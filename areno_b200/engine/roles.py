"""Auxiliary model roles on a rank worker: frozen reference, trainable critic, frozen reward model.

Operations (``areno/engine/roles.py:165-477`` in the reference): ``ensure_roles`` builds roles
(copying the actor's weights when a role points at the actor checkpoint instead of re-reading it),
``score_logprobs`` (per-token log-probs with a leading 0.0, aligned with the input tokens),
``score_values`` (critic value of every position), ``score_rewards`` (scalar at the last token) and
``train_values`` (clipped value loss, one optimizer step per accumulation group).

Differences: rows are scored as packed variable-length batches under a token budget (no padding
FLOPs); roles stay resident on the GPU while they fit (180 GB of HBM holds a 7B actor with its
optimizer state next to a frozen 7B reference) and are swapped through host memory only under
memory pressure, where the reference offloads and reloads full weights on every role call.
"""

from __future__ import annotations

import json
import os
from typing import Any

import torch

from ..models import registry as model_registry
from ..models.dense import TrainMeta
from ..ops.attention import build_varlen_meta
from ..parallel.context import get_context
from ..utils.log import get_logger
from .config import OptimizerConfig
from .logprobs import lm_head_logprobs
from .optim import ShardedAdamW
from .training import to_device

logger = get_logger()

_HEAD_KEYS = ("score.weight", "v_head.summary.weight", "v_head.weight", "value_head.weight", "classifier.weight",
              "reward_head.weight", "regression_head.weight")


def canonical_model_path(path: str | None) -> str | None:
    return os.path.realpath(path) if path else None


def find_head_tensors(path: str) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    """Locate a scalar head (weight, optional bias) in a HF safetensors checkpoint by common key names."""
    from safetensors import safe_open

    files = []
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f).get("weight_map", {})
        for key in _HEAD_KEYS:
            if key in wm:
                files.append((key, os.path.join(path, wm[key])))
    elif os.path.exists(os.path.join(path, "model.safetensors")):
        files = [(k, os.path.join(path, "model.safetensors")) for k in _HEAD_KEYS]
    for key, fname in files:
        try:
            with safe_open(fname, framework="pt") as f:
                keys = set(f.keys())
                if key in keys:
                    w = f.get_tensor(key)
                    bkey = key[: -len("weight")] + "bias"
                    return w, (f.get_tensor(bkey) if bkey in keys else None)
        except (OSError, ValueError):
            continue
    return None, None


class WorkerRole:
    def __init__(self, name: str, path: str, model, value_head, optimizer):
        self.name, self.path, self.model, self.value_head, self.optimizer = name, path, model, value_head, optimizer
        self.on_device = True

    def parameters(self):
        yield from self.model.parameters()
        if self.value_head is not None:
            yield from self.value_head.parameters()

    def offload(self) -> None:
        if not self.on_device:
            return
        self.model.offload_train_weights()
        if self.value_head is not None:
            self.value_head.to("cpu")
        if self.optimizer is not None:
            self.optimizer.offload_state()
        self.on_device = False

    def onload(self, device) -> None:
        if self.on_device:
            return
        self.model.onload_train_weights(device)
        if self.value_head is not None:
            self.value_head.to(device)
        if self.optimizer is not None:
            self.optimizer.onload_state(device)
        self.on_device = True


class _RoleModule(torch.nn.Module):
    """Model + value head as one module so a single sharded optimizer covers both."""

    def __init__(self, model, head):
        super().__init__()
        self.model, self.head = model, head


class RoleManager:
    def __init__(self, worker):
        self.worker = worker
        self.roles: dict[str, WorkerRole] = {}
        self.score_token_budget = 16384

    # ----------------------------------------------------------------- set-up
    def ensure_roles(self, roles: dict[str, Any]) -> None:
        w = self.worker
        actor_path = canonical_model_path(w.config.model_path)
        sources: dict[str, torch.nn.Module] = {}
        if actor_path:
            sources[actor_path] = w.model
        for r in self.roles.values():
            p = canonical_model_path(r.path)
            if p:
                sources.setdefault(p, r.model)
        for name, spec in roles.items():
            if name == "actor" or name in self.roles:
                continue
            role = self._build_role(name, spec, sources)
            self.roles[name] = role
            p = canonical_model_path(spec.path)
            if p:
                sources.setdefault(p, role.model)
            self._maybe_evict(keep=None)

    def _build_role(self, name: str, spec, sources) -> WorkerRole:
        w = self.worker
        path = spec.path
        same_as_actor = (not path) or canonical_model_path(path) == canonical_model_path(w.config.model_path)
        if path and os.path.exists(os.path.join(path, "config.json")):
            adapter, mcfg = model_registry.config_from_pretrained(path)
        else:
            adapter, mcfg = w.adapter, w.config.model
        model = adapter.build(mcfg, device=w.device)
        src = sources.get(canonical_model_path(path)) if path else None
        if src is None and same_as_actor:
            src = w.model
        if src is not None:
            with torch.no_grad():
                for dst_p, src_p in zip(model.parameters(), src.parameters()):
                    dst_p.copy_(src_p.to(dst_p.device))
        elif w.config.dummy_load:
            adapter.init_random(model, seed=w.config.seed + 17)
        else:
            adapter.load_weights(model, path, mcfg)
        head = None
        if name in ("critic", "reward"):
            hw, hb = (find_head_tensors(path) if path and os.path.isdir(path) else (None, None))
            out = int(hw.shape[0]) if hw is not None else 1
            head = torch.nn.Linear(mcfg.hidden_size, out, bias=hb is not None, dtype=mcfg.dtype, device=w.device)
            with torch.no_grad():
                if hw is not None:
                    head.weight.copy_(hw.to(head.weight))
                    if hb is not None:
                        head.bias.copy_(hb.to(head.bias))
                elif name == "reward":
                    raise ValueError(f"reward checkpoint {path!r} has no scalar head ({', '.join(_HEAD_KEYS)})")
                else:
                    head.weight.zero_()
            for p in head.parameters():
                p.tp_replicated_grad = "same"     # scalar head on the replicated hidden state: same gradient on every rank
        optimizer = None
        if spec.trainable:
            ocfg = OptimizerConfig(**{**w.config.optimizer.__dict__})
            if spec.optimizer_lr is not None:
                ocfg.lr = float(spec.optimizer_lr)
            ocfg.lr_decay_style = "constant"
            optimizer = ShardedAdamW(_RoleModule(model, head) if head is not None else model, ocfg)
        else:
            for p in model.parameters():
                p.requires_grad_(False)
        logger.info("role=%s stage=built trainable=%s head=%s source=%s", name, bool(spec.trainable), head is not None,
                    "actor-copy" if src is not None else (path or "random"))
        return WorkerRole(name, path, model, head, optimizer)

    # ------------------------------------------------------------- residency
    def _free_bytes(self) -> int:
        if self.worker.device.type != "cuda":
            return 1 << 62
        free, _ = torch.cuda.mem_get_info(self.worker.device)
        return free + torch.cuda.memory_reserved(self.worker.device) - torch.cuda.memory_allocated(self.worker.device)

    def _maybe_evict(self, keep: str | None, need: int = 24 << 30) -> None:
        """Under memory pressure move idle roles (then the actor) to the host."""
        if self._free_bytes() >= need:
            return
        for name, role in self.roles.items():
            if name != keep and role.on_device:
                role.offload()
                if self.worker.device.type == "cuda":
                    torch.cuda.empty_cache()
                if self._free_bytes() >= need:
                    return
        if keep != "actor":
            self.worker.prepare_actor_offloaded()

    def _activate(self, name: str):
        w = self.worker
        if name == "actor":
            w.prepare_actor_onloaded()
            return w.model, None
        role = self.roles[name]
        if not role.on_device:
            self._maybe_evict(keep=name, need=40 << 30)
            role.onload(w.device)
        else:
            self._maybe_evict(keep=name)
        return role.model, role

    # ---------------------------------------------------------------- scoring
    def _microbatches(self, rows: list[list[int]], microbatch_size: int):
        cur, tokens = [], 0
        for i, r in enumerate(rows):
            if cur and (len(cur) >= max(microbatch_size, 1) * 8 or tokens + len(r) > self.score_token_budget):
                yield cur
                cur, tokens = [], 0
            cur.append(i)
            tokens += len(r)
        if cur:
            yield cur

    def _ep_aligned(self, model, rows, microbatches):
        """Expert parallelism: the ranks score different rows in different numbers of micro-batches, but every
        forward pass is a group-wide exchange.  The ranks agree on the number of rounds and on the largest
        micro-batch of each; a rank that has run out of rows takes part with an idle pass.  Yields the local
        micro-batches (index lists) with the round's communicator size pinned."""
        from ..parallel.context import get_context

        ctx = get_context()
        if ctx.ep_size <= 1 or not hasattr(model, "ep_idle_forward"):
            yield from microbatches
            return
        rt = ctx.ep_runtime
        mbs = list(microbatches)
        sizes = [sum(max(len(rows[i]), 1) for i in idx) for idx in mbs]
        rounds = rt.agree_max([len(mbs)])[0]
        if rounds == 0:
            return
        caps = rt.agree_max(sizes + [0] * (rounds - len(sizes)))
        for r in range(rounds):
            with rt.pinned(caps[r]):
                if r < len(mbs):
                    yield mbs[r]
                else:
                    model.ep_idle_forward()

    def _packed_forward(self, model, rows: list[list[int]]):
        dev = self.worker.device
        lens = [max(len(r), 1) for r in rows]
        flat = [t for r in rows for t in (r if r else [0])]
        ids = torch.tensor(flat, dtype=torch.int64)
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
        if dev.type == "cuda":
            ids, pos = ids.pin_memory().to(dev, non_blocking=True), pos.pin_memory().to(dev, non_blocking=True)
        meta = TrainMeta(build_varlen_meta(lens, device=dev), activation_checkpointing=False)
        return model(ids, pos, meta).hidden_states, ids, lens

    @torch.no_grad()
    def score_logprobs(self, role: str, rows: list[list[int]], pad_token_id: int = 0, microbatch_size: int = 8):
        model, _ = self._activate(role)
        model.eval()
        out: list[list[float]] = [[] for _ in rows]
        for idx in self._ep_aligned(model, rows, self._microbatches(rows, microbatch_size)):
            sub = [rows[i] for i in idx]
            hidden, ids, lens = self._packed_forward(model, sub)
            starts = [0]
            for n in lens:
                starts.append(starts[-1] + n)
            act = torch.cat([torch.arange(starts[j], starts[j + 1] - 1) for j in range(len(sub))]).to(hidden.device)
            if act.numel():
                lp = lm_head_logprobs(model.lm_head, hidden.index_select(0, act), ids.index_select(0, act + 1),
                                      self.worker.config.runtime.logprob_chunk,
                                      softcap=model.cfg.final_logit_softcapping).float().cpu().tolist()
            else:
                lp = []
            k = 0
            for j, i in enumerate(idx):
                n = lens[j]
                out[i] = [0.0] + lp[k:k + n - 1]
                k += n - 1
        return out

    @torch.no_grad()
    def score_values(self, role: str, rows: list[list[int]], pad_token_id: int = 0, microbatch_size: int = 8):
        model, r = self._activate(role)
        if r is None or r.value_head is None:
            raise RuntimeError(f"role {role!r} has no value head")
        model.eval()
        out: list[list[float]] = [[] for _ in rows]
        for idx in self._ep_aligned(model, rows, self._microbatches(rows, microbatch_size)):
            sub = [rows[i] for i in idx]
            hidden, _ids, lens = self._packed_forward(model, sub)
            values = r.value_head(hidden)
            values = (values.squeeze(-1) if values.shape[-1] == 1 else values[..., -1]).float().cpu().tolist()
            k = 0
            for j, i in enumerate(idx):
                out[i] = values[k:k + lens[j]]
                k += lens[j]
        return out

    @torch.no_grad()
    def score_rewards(self, role: str, rows: list[list[int]], pad_token_id: int = 0, microbatch_size: int = 8):
        per_token = self.score_values(role, rows, pad_token_id, microbatch_size)
        return [float(v[-1]) if v else 0.0 for v in per_token]

    # --------------------------------------------------------------- training
    def train_values(self, role: str, packs: list, gradient_accumulation_steps: int | None = None, *,
                     cliprange_value: float = 0.5, value_loss_coef: float = 0.5) -> dict:
        ctx = get_context()
        model, r = self._activate(role)
        if r is None or r.value_head is None or r.optimizer is None:
            raise RuntimeError(f"role {role!r} is not a trainable value model")
        model.train()
        rows = [p[ctx.dp_rank] if isinstance(p, (list, tuple)) else p for p in packs]
        accum = len(rows) if not gradient_accumulation_steps else max(int(gradient_accumulation_steps), 1)
        stats = _CriticStats()
        for i, pack in enumerate(rows):
            g0 = (i // accum) * accum
            group = min(accum, len(rows) - g0)
            last = (i + 1) % accum == 0 or i == len(rows) - 1
            self._value_microbatch(r, pack, cliprange_value, value_loss_coef, group, stats)
            if last:
                r.optimizer.step(lr=r.optimizer.lr, clip_norm=self.worker.config.optimizer.grad_clip_norm)
        return stats.to_dict()

    def _value_microbatch(self, role: WorkerRole, pack: dict, clip: float, coef: float, group: int, stats) -> None:
        dev = self.worker.device
        pack = to_device({k: v for k, v in pack.items() if isinstance(v, torch.Tensor)}, dev)
        ids2d = pack["input_ids"].long()
        lengths = pack["lengths"].long().clamp(min=1, max=ids2d.shape[1])
        width = ids2d.shape[1]
        valid_tok = torch.arange(width, device=dev)[None, :] < lengths[:, None]
        ids = ids2d[valid_tok]
        pos = torch.arange(width, device=dev, dtype=torch.int32)[None, :].expand_as(ids2d)[valid_tok]
        meta = TrainMeta(build_varlen_meta(lengths.tolist(), device=dev),
                         activation_checkpointing=self.worker.config.runtime.activation_checkpointing)
        hidden = role.model(ids, pos, meta).hidden_states
        values = role.value_head(hidden).squeeze(-1).float()          # packed [T]
        # position t is trained when token t+1 exists and is a response token
        nxt = torch.zeros_like(valid_tok)
        nxt[:, :-1] = valid_tok[:, 1:] & ~pack["prompt_mask"].bool()[:, 1:]
        target2d = torch.zeros_like(pack["returns"].float())
        target2d[:, :-1] = pack["returns"].float()[:, 1:]
        base2d = torch.zeros_like(target2d)
        base2d[:, :-1] = pack["values"].float()[:, 1:]
        mask, target, base = nxt[valid_tok], target2d[valid_tok], base2d[valid_tok]
        if not bool(mask.any()):
            (values.sum() * 0.0).backward()
            return
        clipped = base + (values - base).clamp(-clip, clip)
        l_un, l_cl = (values - target).pow(2), (clipped - target).pow(2)
        loss = coef * 0.5 * torch.maximum(l_un[mask], l_cl[mask]).mean()
        (loss / max(group, 1)).backward()
        stats.add(loss, l_un[mask], l_cl[mask], values[mask], target[mask], base[mask])


class _CriticStats:
    KEYS = ("critic_value_loss", "critic_value_clipfrac", "critic_value_mse", "critic_value_pred_mean",
            "critic_value_target_mean", "critic_old_value_mean", "critic_value_abs_error_mean")

    def __init__(self):
        self.rows: list[torch.Tensor] = []

    def add(self, loss, l_un, l_cl, pred, target, base) -> None:
        with torch.no_grad():
            self.rows.append(torch.stack([loss.detach().float(), (l_cl > l_un).float().mean(), l_un.mean(), pred.mean(),
                                          target.mean(), base.mean(), (pred - target).abs().mean()]))

    def to_dict(self) -> dict[str, float]:
        if not self.rows:
            return {k: 0.0 for k in self.KEYS}
        mean = torch.stack(self.rows).mean(0).cpu().tolist()
        return dict(zip(self.KEYS, (float(v) for v in mean)))
