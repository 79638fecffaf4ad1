"""DP-sharded AdamW over flat parameter / gradient buckets.

Layout: parameters are re-pointed into flat bf16 buffers ("buckets", reverse registration order so
the last layers - whose gradients arrive first in backward - fill the first buckets) and each
gets an fp32 ``main_grad`` view into a matching flat gradient buffer that the wgrad GEMM epilogue,
the norm backward and the embedding backward accumulate into directly.  Every DP rank owns the
``1/dp`` slice of each bucket: after the last micro-batch the bucket's gradient is
reduce-scattered in place, the fused AdamW kernel updates the rank's fp32 master / moment shard and
writes the bf16 shard, and the bucket's parameters are all-gathered in place.  Gradients,
optimizer state and the update are sharded; only the bf16 working copy is replicated.

Numerics follow the reference optimizer (``areno/engine/optim/adamw_fp32_master.py:239-303``,
``adamw_8bit.py``): decoupled decay on every parameter, eps outside the square root, bias
correction by step count, fp32 gradient accumulation, clip coefficient ``max_norm / (norm + 1e-6)``.
The 8-bit variant keeps int8/uint8 moments with one scale per 32 elements and no master copy.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..ops import optim as optim_ops
from ..parallel.context import ParallelContext, get_context
from ..utils.tracing import trace_range
from .config import OptimizerConfig

_ALIGN = 256  # elements; keeps every shard boundary 16-byte aligned for all dtypes


def _tp_grad_kind(p) -> str:
    """How a parameter's gradient relates to the TP group, from its ``tp_replicated_grad`` annotation.

    ``"sharded"``  no annotation: the parameter is a TP shard and its gradient is complete.
    ``"partial"``  ``True``: the parameter is replicated and each rank computed the part of the gradient that
                   flows through its own heads / experts; the ranks' gradients are summed.
    ``"same"``     ``"same"``: replicated, and every rank already holds the full gradient because the gradient
                   of the parameter's output was summed upstream (norm scales in front of a column-parallel
                   layer, biases added after a row-parallel reduce, scalar heads on the replicated hidden
                   state); nothing is reduced, and the norm counts it once.
    """
    flag = getattr(p, "tp_replicated_grad", False)
    if flag == "same":
        return "same"
    return "partial" if flag else "sharded"


@dataclass
class _Bucket:
    params: list = field(default_factory=list)
    offsets: list = field(default_factory=list)
    numel: int = 0            # padded
    replicated: bool = False  # parameters replicated over TP (norm scales, biases of row-parallel layers)
    tp_sum: bool = False      # replicated, and each TP rank holds only its part of the gradient (sum over TP needed)
    param_flat: torch.Tensor | None = None
    grad_flat: torch.Tensor | None = None
    master: torch.Tensor | None = None
    m: torch.Tensor | None = None
    v: torch.Tensor | None = None
    m_scale: torch.Tensor | None = None
    v_scale: torch.Tensor | None = None
    shard: int = 0
    grad_offset: int = 0      # element offset of grad_flat inside the symmetric gradient region (peer-memory path)
    min_layer: int = -1       # lowest decoder-layer index among the parameters (-1: embeddings and the like)
    # expert-parallel parameters: every data-parallel rank owns different experts, whose gradient is already the
    # sum over all ranks' tokens.  The bucket is not sharded (shard == numel), never reduced and never gathered.
    local: bool = False


class ShardedAdamW:
    def __init__(self, model: torch.nn.Module, cfg: OptimizerConfig, ctx: ParallelContext | None = None,
                 sequence_parallel: bool = False):
        """``sequence_parallel``: the model runs its norms and residual stream on 1 / tp of the rows, so replicated
        parameters annotated ``"same"`` (norm scales, row-parallel biases) only see their own rows' gradient and are
        summed over TP like the ``partial`` ones."""
        self.cfg = cfg
        self.sequence_parallel = bool(sequence_parallel)
        self.ctx = ctx or get_context()
        self.dp = max(1, self.ctx.dp_size)
        self.dp_rank = self.ctx.dp_rank
        self.step_count = 0
        self.lr = cfg.lr
        self.buckets: list[_Bucket] = []
        self._state_ready = False
        self.grad_comm = None       # parallel.grad_comm.GradComm when gradients are reduced over peer memory
        self._overlap = False
        self._build(model)

    # ------------------------------------------------------------------ layout
    def _build(self, model):
        seen = set()
        params = []
        for p in model.parameters():
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                params.append(p)
        params.reverse()
        cap = max(int(self.cfg.fp32_master_bucket_numel), 1)
        granule = _ALIGN * self.dp
        # one bucket family per (TP-replicated?, dtype): fp32 parameters (router gates, decay rates, conv
        # taps) keep their precision instead of being folded into a bf16 buffer
        groups: dict[tuple, list] = {}
        for p in params:
            groups.setdefault((_tp_grad_kind(p), p.dtype, bool(getattr(p, "ep_local", False))), []).append(p)
        for (kind, _dtype, local), plist in groups.items():
            replicated = kind != "sharded"
            tp_sum = kind == "partial" or (kind == "same" and self.sequence_parallel)
            cur = _Bucket(replicated=replicated, tp_sum=tp_sum, local=local)
            for p in plist:
                n = (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
                if cur.params and cur.numel + n > cap:
                    self.buckets.append(cur)
                    cur = _Bucket(replicated=replicated, tp_sum=tp_sum, local=local)
                cur.params.append(p)
                cur.offsets.append(cur.numel)
                cur.numel += n
            if cur.params:
                self.buckets.append(cur)
        layer_of = _layer_index_of(model)
        off = 0
        for b in self.buckets:
            b.min_layer = min(layer_of.get(id(p), -1) for p in b.params)
            if b.local:
                b.shard = b.numel
                continue
            b.numel = (b.numel + granule - 1) // granule * granule
            b.shard = b.numel // self.dp
            b.grad_offset = off
            off += b.numel
        self.grad_comm = self._make_grad_comm(off)
        for b in self.buckets:
            dev = b.params[0].device
            dtype = b.params[0].dtype
            b.param_flat = torch.zeros(b.numel, dtype=dtype, device=dev)
            if self.grad_comm is not None and not b.local:
                b.grad_flat = self.grad_comm.view(b.grad_offset, b.numel)
            else:
                b.grad_flat = torch.zeros(b.numel, dtype=torch.float32, device=dev)
            for p, off in zip(b.params, b.offsets):
                view = b.param_flat[off:off + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = b.grad_flat[off:off + p.numel()].view(p.shape)
                p.grad_added_to_main_grad = False

    def _lo(self, b: _Bucket) -> int:
        """First element of this rank's shard of the bucket."""
        return 0 if b.local else self.dp_rank * b.shard

    def _make_grad_comm(self, total_elems: int):
        """Peer-memory gradient reduce-scatter: CUDA, more than one DP rank, at most 8 (one NVLink domain).
        ``ARENO_FUSED_GRAD_RS=0`` keeps the NCCL reduce-scatter."""
        dev = self.buckets[0].params[0].device if self.buckets else None
        if (self.dp <= 1 or total_elems <= 0 or self.dp > 8 or dev is None or dev.type != "cuda" or len(self.buckets) > 4096
                or os.environ.get("ARENO_FUSED_GRAD_RS", "1") == "0"):
            return None
        from ..parallel.grad_comm import GradComm

        comm, err = None, None
        try:
            comm = GradComm(self.ctx.dp_group, self.dp, self.dp_rank, total_elems, dev)
        except Exception as exc:  # e.g. peer access unavailable: every rank must then take the NCCL path
            err = exc
        ok = torch.tensor([0 if comm is None else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.ctx.dp_group)
        if int(ok.item()) == 0:
            if comm is not None:
                comm.close()
            if err is not None:
                import logging

                logging.getLogger("areno").warning("peer-memory gradient reduce-scatter unavailable (%s); using NCCL", err)
            return None
        return comm

    # ------------------------------------------------- overlap with backward
    def begin_overlap(self):
        """Arm the reduction for the micro-batch whose backward ends the accumulation window.  Returns the
        hook to pass as ``TrainMeta.layer_grad_hook`` (``None`` when gradients go through NCCL)."""
        if self.grad_comm is None or self.ctx.tp_size > 1:
            return None
        self.grad_comm.begin_step()
        self._overlap = True
        return self.on_layer_grad_done

    def on_layer_grad_done(self, layer: int) -> None:
        """Backward has passed decoder layer ``layer``: every bucket made only of later parameters is final."""
        if not self._overlap:
            return
        for i, b in enumerate(self.buckets):
            if not b.local and b.min_layer >= layer and i not in self.grad_comm.launched:
                self._fold_bucket(b)
                self.grad_comm.launch(i, b.grad_offset, b.shard)

    @staticmethod
    def _fold_bucket(b: _Bucket) -> None:
        for p in b.params:
            if p.grad is not None:
                if not getattr(p, "grad_added_to_main_grad", False):
                    p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None
            p.grad_added_to_main_grad = False

    def _ensure_state(self):
        if self._state_ready:
            return
        for b in self.buckets:
            lo = self._lo(b)
            dev = b.param_flat.device
            if b.param_flat.dtype == torch.float32:
                # fp32 parameters are their own master copy: the update runs in place on the local shard
                b.master = b.param_flat[lo:lo + b.shard]
                b.m = torch.zeros(b.shard, dtype=torch.float32, device=dev)
                b.v = torch.zeros(b.shard, dtype=torch.float32, device=dev)
            elif self.cfg.adam_8bit:
                nb = (b.shard + optim_ops.Q_BLOCK - 1) // optim_ops.Q_BLOCK
                b.m = torch.zeros(b.shard, dtype=torch.int8, device=dev)
                b.v = torch.zeros(b.shard, dtype=torch.uint8, device=dev)
                b.m_scale = torch.full((nb,), 1e-30, dtype=torch.float32, device=dev)
                b.v_scale = torch.full((nb,), 1e-30, dtype=torch.float32, device=dev)
            else:
                b.master = b.param_flat[lo:lo + b.shard].float()
                b.m = torch.zeros(b.shard, dtype=torch.float32, device=dev)
                b.v = torch.zeros(b.shard, dtype=torch.float32, device=dev)
        self._state_ready = True

    # -------------------------------------------------------------- gradients
    def fold_param_grads(self):
        """Accumulate any autograd-produced ``p.grad`` (ops without a fused main-grad path) into the
        fp32 buffers and drop it."""
        for b in self.buckets:
            for p in b.params:
                if p.grad is not None:
                    if not getattr(p, "grad_added_to_main_grad", False):
                        p.main_grad.add_(p.grad.to(torch.float32))
                    p.grad = None
                p.grad_added_to_main_grad = False

    def zero_grad(self):
        for b in self.buckets:
            b.grad_flat.zero_()
            for p in b.params:
                p.grad = None
                p.grad_added_to_main_grad = False

    def _grad_shard(self, b: _Bucket) -> torch.Tensor:
        lo = self._lo(b)
        return b.grad_flat[lo:lo + b.shard]

    def reduce_gradients(self):
        """TP all-reduce of the replicated parameters whose ranks hold partial gradients, then DP reduce-scatter (sum)
        in place."""
        ctx = self.ctx
        if ctx.tp_size > 1:
            for b in self.buckets:
                if b.tp_sum:      # "same" buckets already hold the full gradient on every rank
                    dist.all_reduce(b.grad_flat, group=ctx.tp_group)
            self._sum_replicated_kv_grads()
        if self.dp > 1 and self.grad_comm is not None:
            if not self._overlap:
                self.grad_comm.begin_step()
            for i, b in enumerate(self.buckets):     # whatever backward did not hand over yet
                if not b.local:
                    self.grad_comm.launch(i, b.grad_offset, b.shard)
            self.grad_comm.finish()
            self._overlap = False
        elif self.dp > 1:
            works = []
            for b in self.buckets:
                if b.local:
                    continue
                works.append(dist.reduce_scatter_tensor(self._grad_shard(b), b.grad_flat, group=ctx.dp_group,
                                                        async_op=True))
            for w in works:
                w.wait()

    @torch.no_grad()
    def self_check_reduce_scatter(self, bucket: int = 0) -> float | None:
        """Reduce one bucket of random gradients with the peer-memory kernel and with NCCL's
        ``reduce_scatter_tensor`` and return the largest absolute difference on this rank's shard (``None`` when the
        NCCL path is in use).  Must be called between steps (the bucket is zeroed afterwards)."""
        if self.grad_comm is None or self.dp <= 1 or not self.buckets:
            return None
        shared = [x for x in self.buckets if not x.local]
        if not shared:
            return None
        b = shared[min(bucket, len(shared) - 1)]
        i = self.buckets.index(b)
        g = torch.Generator(device=b.grad_flat.device).manual_seed(4321 + self.dp_rank)
        b.grad_flat.copy_(torch.randn(b.grad_flat.shape, device=b.grad_flat.device, generator=g))
        want = torch.empty(b.shard, dtype=torch.float32, device=b.grad_flat.device)
        dist.reduce_scatter_tensor(want, b.grad_flat.clone(), group=self.ctx.dp_group)
        self.grad_comm.begin_step()
        self.grad_comm.launch(i, b.grad_offset, b.shard)
        self.grad_comm.finish()
        err = float((self._grad_shard(b) - want).abs().max())
        torch.cuda.synchronize()
        dist.barrier(group=self.ctx.dp_group)       # nobody zeroes the bucket while a peer may still be reading it
        b.grad_flat.zero_()
        return err

    def _sum_replicated_kv_grads(self):
        """K / V rows of a fused qkv projection are copies of one another on ``rep`` neighbouring ranks when the TP
        size exceeds the KV head count (``kv_replicated`` on the parameter).  Each copy only sees the gradient of
        its own query heads; summing over the copies keeps them identical."""
        ctx = self.ctx
        tp = ctx.tp_size
        for b in self.buckets:
            for p, off in zip(b.params, b.offsets):
                rep = int(getattr(p, "kv_replicated", 0) or 0)
                if rep <= 1:
                    continue
                hq_rows, _hkv, d, _ = p.tp_shard[1]
                inner = p.numel() // p.shape[0]
                g = b.grad_flat[off + hq_rows * d * inner: off + p.numel()]
                buf = g.new_zeros((tp // rep, g.numel()))
                buf[ctx.tp_rank // rep].copy_(g)
                dist.all_reduce(buf, group=ctx.tp_group)
                g.copy_(buf[ctx.tp_rank // rep])

    def grad_norm_sq(self) -> torch.Tensor:
        """Squared global gradient norm (of the DP-averaged gradient) as a 1-element device tensor."""
        ctx = self.ctx
        dev = self.buckets[0].grad_flat.device
        sharded = torch.zeros(1, dtype=torch.float32, device=dev)
        repl = torch.zeros(1, dtype=torch.float32, device=dev)
        for b in self.buckets:
            optim_ops.sumsq(self._grad_shard(b), repl if b.replicated else sharded, accumulate=True)
            if ctx.tp_size > 1 and not b.replicated:
                # K / V rows that exist on `rep` ranks would be counted `rep` times by the TP sum below
                lo = self._lo(b)
                for p, off in zip(b.params, b.offsets):
                    rep = int(getattr(p, "kv_replicated", 0) or 0)
                    if rep > 1:
                        hq_rows, _hkv, d, _ = p.tp_shard[1]
                        a0 = max(off + hq_rows * d * (p.numel() // p.shape[0]), lo)
                        a1 = min(off + p.numel(), lo + b.shard)
                        if a1 > a0:
                            sharded -= b.grad_flat[a0:a1].pow(2).sum() * ((rep - 1) / rep)
        total = sharded + repl / max(1, ctx.tp_size)
        total = total / float(self.dp * self.dp)
        if self.dp > 1:
            dist.all_reduce(total, group=ctx.dp_group)
        if ctx.tp_size > 1:
            dist.all_reduce(total, group=ctx.tp_group)
        return total

    # ------------------------------------------------------------------- step
    def step(self, lr: float | None = None, clip_norm: float | None = None) -> torch.Tensor:
        """Reduce, clip, update, all-gather.  Returns the gradient norm (device scalar tensor)."""
        self._ensure_state()
        self.fold_param_grads()
        with trace_range("optimizer/reduce_gradients"):
            self.reduce_gradients()
        lr = self.lr if lr is None else lr
        with trace_range("optimizer/grad_norm"):
            norm = torch.sqrt(self.grad_norm_sq())
        coef = None
        clip = self.cfg.grad_clip_norm if clip_norm is None else clip_norm
        if clip is not None and clip > 0:
            coef = torch.clamp(clip / (norm + 1e-6), max=1.0)
        self.step_count += 1
        b1, b2 = self.cfg.betas
        gathers = []
        for b in self.buckets:
            lo = self._lo(b)
            g = self._grad_shard(b)
            out = b.param_flat[lo:lo + b.shard]
            if b.param_flat.dtype == torch.float32:
                optim_ops.adamw_fp32(b.master, b.m, b.v, g, None, lr, b1, b2, self.cfg.eps, self.cfg.weight_decay,
                                     self.step_count, 1.0 / self.dp, coef)
            elif self.cfg.adam_8bit:
                optim_ops.adamw_8bit(None, b.m, b.v, b.m_scale, b.v_scale, g, out, lr, b1, b2, self.cfg.eps,
                                     self.cfg.weight_decay, self.step_count, 1.0 / self.dp, coef)
            else:
                optim_ops.adamw_fp32(b.master, b.m, b.v, g, out, lr, b1, b2, self.cfg.eps, self.cfg.weight_decay,
                                     self.step_count, 1.0 / self.dp, coef)
            if self.dp > 1 and not b.local:
                gathers.append(dist.all_gather_into_tensor(b.param_flat, out, group=self.ctx.dp_group, async_op=True))
        with trace_range("optimizer/param_all_gather_wait"):
            for w in gathers:
                w.wait()
        self.zero_grad()
        return norm

    # --------------------------------------------------------------- offload
    def offload_state(self):
        for b in self.buckets:
            own_master = b.param_flat is not None and b.param_flat.dtype == torch.float32
            for name in ("master", "m", "v", "m_scale", "v_scale", "grad_flat"):
                if name == "master" and own_master:
                    b.master = None   # a view of the parameters themselves: rebuilt on onload
                    continue
                if name == "grad_flat" and self.grad_comm is not None:
                    continue          # lives in the peer-mapped region, which stays on the device
                t = getattr(b, name)
                if t is not None and t.is_cuda:
                    setattr(b, name, t.to("cpu"))
        self._offloaded = True

    def onload_state(self, device):
        for b in self.buckets:
            for name in ("master", "m", "v", "m_scale", "v_scale", "grad_flat"):
                t = getattr(b, name)
                if t is not None and not t.is_cuda:
                    setattr(b, name, t.to(device))
            for p, off in zip(b.params, b.offsets):
                p.main_grad = b.grad_flat[off:off + p.numel()].view(p.shape)
            if self._state_ready and b.master is None and b.param_flat.dtype == torch.float32:
                lo = self._lo(b)
                b.master = b.param_flat[lo:lo + b.shard]
        self._offloaded = False

    # ------------------------------------------------------------ state dict
    def state_dict(self) -> dict:
        self._ensure_state()
        return {
            "step": self.step_count,
            "dp_rank": self.dp_rank,
            "dp_size": self.dp,
            "adam_8bit": self.cfg.adam_8bit,
            "buckets": [
                {k: (getattr(b, k).detach().cpu() if getattr(b, k) is not None else None)
                 for k in ("master", "m", "v", "m_scale", "v_scale")}
                for b in self.buckets
            ],
        }

    def load_state_dict(self, state: dict) -> None:
        self._ensure_state()
        if state.get("dp_size") != self.dp or len(state["buckets"]) != len(self.buckets):
            raise ValueError("optimizer state was saved with a different sharding layout")
        self.step_count = int(state["step"])
        for b, sb in zip(self.buckets, state["buckets"]):
            for k, t in sb.items():
                if t is not None:
                    getattr(b, k).copy_(t)


def _layer_index_of(model) -> dict[int, int]:
    """``id(parameter) -> decoder layer index``; final norm / LM head count as one past the last layer
    (their gradients are the first to be final in backward), everything else (embeddings, per-layer input
    tables) as -1 (final only when backward ends)."""
    out: dict[int, int] = {}
    n_layers = len(getattr(model, "layers", []) or [])
    for name, p in model.named_parameters():
        if id(p) in out:
            continue
        parts = name.split(".")
        if parts[0] == "layers" and len(parts) > 1 and parts[1].isdigit():
            out[id(p)] = int(parts[1])
        elif parts[0] in ("norm", "lm_head"):
            out[id(p)] = n_layers
        else:
            out[id(p)] = -1
    return out


def lr_for_step(cfg: OptimizerConfig, step: int) -> float:
    """Warm-up then constant / linear / cosine decay to ``min_lr`` over ``lr_decay_steps``
    (schedule of ``areno/engine/training.py:138-155``); ``step`` counts from 1."""
    lr, min_lr = cfg.lr, cfg.min_lr
    if cfg.lr_warmup_steps > 0 and step <= cfg.lr_warmup_steps:
        return lr * step / cfg.lr_warmup_steps
    if cfg.lr_decay_style == "constant" or cfg.lr_decay_steps <= 0:
        return lr
    span = max(cfg.lr_decay_steps - cfg.lr_warmup_steps, 1)
    t = min(max((step - cfg.lr_warmup_steps) / span, 0.0), 1.0)
    if cfg.lr_decay_style == "linear":
        return min_lr + (lr - min_lr) * (1.0 - t)
    if cfg.lr_decay_style == "cosine":
        return min_lr + (lr - min_lr) * 0.5 * (1.0 + math.cos(math.pi * t))
    raise ValueError(f"unknown lr_decay_style {cfg.lr_decay_style}")
