"""Process-group layout: ``global_rank = dp_rank * tp_size + tp_rank``; one TP group per DP row and
one DP group per TP column (same layout as ``areno/engine/parallel/context.py:65-127``).  NCCL on
CUDA, Gloo on CPU; rendezvous over TCP on 127.0.0.1.

A job may use two layouts over the same ranks: the training layout (the installed context) and a
rollout layout with a different TP width (``ctx.rollout``), e.g. training as pure data parallel with
sharded optimizer state while decoding tensor-parallel so that every weight byte is read once per
TP group instead of once per GPU.  Code that must run in the rollout layout wraps itself in
``use_context(ctx.rollout)``."""

from __future__ import annotations

import contextlib
import datetime
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist


@dataclass
class ParallelContext:
    rank: int = 0
    world_size: int = 1
    tp_rank: int = 0
    tp_size: int = 1
    dp_rank: int = 0
    dp_size: int = 1
    tp_group: Any = None
    dp_group: Any = None
    device: torch.device = torch.device("cpu")
    rollout: "ParallelContext | None" = None  # second layout for the inference engine (None: same as training)
    # Expert parallelism: the experts of a mixture-of-experts layer are dealt out over the data-parallel group
    # (every rank keeps its own tokens and E / ep_size experts); requires tp_size == 1.  ``ep_ctl_group`` is a
    # CPU (gloo) group over the same ranks for the host-side agreements of the engine loop; ``ep_runtime`` owns
    # the communicators (parallel/ep.py) once a model that needs them exists.
    ep_size: int = 1
    ep_rank: int = 0
    ep_group: Any = None
    ep_ctl_group: Any = None
    ep_runtime: Any = None

    @property
    def rollout_layout(self) -> "ParallelContext":
        return self.rollout if self.rollout is not None else self


_CONTEXT = ParallelContext()


def get_context() -> ParallelContext:
    return _CONTEXT


def set_context(ctx: ParallelContext) -> None:
    global _CONTEXT
    _CONTEXT = ctx


@contextlib.contextmanager
def use_context(ctx: ParallelContext):
    """Temporarily install ``ctx`` as the global context (layer construction and forward read it)."""
    global _CONTEXT
    prev = _CONTEXT
    _CONTEXT = ctx
    try:
        yield ctx
    finally:
        _CONTEXT = prev


def single_process_context(device: torch.device | str = "cpu") -> ParallelContext:
    ctx = ParallelContext(device=torch.device(device))
    set_context(ctx)
    return ctx


def _layout(rank: int, world_size: int, tp_size: int, backend: str, device) -> ParallelContext:
    """Create the TP / DP sub-groups of one layout (collective: every rank must call it)."""
    if world_size % tp_size != 0:
        raise ValueError(f"world_size {world_size} is not divisible by tp_size {tp_size}")
    dp_size = world_size // tp_size
    tp_group = dp_group = None
    if world_size > 1:
        for d in range(dp_size):
            ranks = list(range(d * tp_size, (d + 1) * tp_size))
            g = dist.new_group(ranks=ranks, backend=backend) if tp_size > 1 else None
            if rank in ranks:
                tp_group = g
        for t in range(tp_size):
            ranks = list(range(t, world_size, tp_size))
            g = dist.new_group(ranks=ranks, backend=backend) if dp_size > 1 else None
            if rank in ranks:
                dp_group = g
    return ParallelContext(rank=rank, world_size=world_size, tp_rank=rank % tp_size, tp_size=tp_size,
                           dp_rank=rank // tp_size, dp_size=dp_size, tp_group=tp_group, dp_group=dp_group,
                           device=device)


def init_parallel(rank: int, world_size: int, tp_size: int, *, master_addr: str = "127.0.0.1", master_port: int = 0,
                  backend: str | None = None, device: torch.device | None = None,
                  timeout_s: float = 1800.0, rollout_tp_size: int | None = None,
                  expert_parallel: bool = False) -> ParallelContext:
    """Create the default group plus TP / DP sub-groups and install the global context.  With
    ``rollout_tp_size`` different from ``tp_size`` a second layout is created as ``ctx.rollout``.  With
    ``expert_parallel`` the data-parallel group doubles as the expert-parallel group (``tp_size`` must be 1)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    if backend is None:
        backend = "nccl" if device.type == "cuda" else "gloo"
    if not dist.is_initialized() and world_size > 1:
        init = f"tcp://{master_addr}:{master_port}" if master_port else "env://"
        kwargs: dict[str, Any] = {}
        if backend == "nccl":
            kwargs["device_id"] = device
        dist.init_process_group(backend=backend, init_method=init, rank=rank, world_size=world_size,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    ctx = _layout(rank, world_size, tp_size, backend, device)
    if rollout_tp_size and rollout_tp_size != tp_size:
        ctx.rollout = _layout(rank, world_size, rollout_tp_size, backend, device)
    if expert_parallel and world_size > 1:
        if tp_size != 1 or ctx.rollout is not None:
            raise ValueError("expert parallelism runs over the data-parallel group: tp_size and rollout_tp_size must be 1")
        ctx.ep_size, ctx.ep_rank, ctx.ep_group = ctx.dp_size, ctx.dp_rank, ctx.dp_group
        # collective: every rank creates the control group (host tensors, so never queued behind GPU work)
        ctx.ep_ctl_group = ctx.dp_group if backend == "gloo" else dist.new_group(ranks=list(range(world_size)),
                                                                                 backend="gloo")
    set_context(ctx)
    return ctx


def destroy_parallel() -> None:
    if dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:
            pass
    set_context(ParallelContext())
