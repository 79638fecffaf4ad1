"""Tensor-parallel collectives as autograd functions (NCCL / Gloo baseline path).

These are the library-collective versions of the TP seams; the fused sm_100a kernels in
``areno_b200.parallel.fused`` replace them on the hot paths when symmetric memory is set up.
Call sites mirror ``areno/engine/parallel/collectives.py:95-242`` of the reference, except that
``reduce_scatter_rows`` is a true reduce-scatter (the reference all-reduces a pre-sliced chunk).
"""

from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

from .context import get_context


def _tp():
    ctx = get_context()
    return ctx.tp_group, ctx.tp_size, ctx.tp_rank


class _ReduceFromTP(torch.autograd.Function):
    """forward: all-reduce (sum); backward: identity."""

    @staticmethod
    def forward(ctx, x):
        group, size, _ = _tp()
        if size == 1:
            return x
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g


class _CopyToTP(torch.autograd.Function):
    """forward: identity; backward: all-reduce (sum)."""

    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        group, size, _ = _tp()
        if size == 1:
            return g
        g = g.contiguous()
        dist.all_reduce(g, group=group)
        return g


class _GatherRows(torch.autograd.Function):
    """forward: all-gather along dim 0; backward: reduce-scatter along dim 0."""

    @staticmethod
    def forward(ctx, x):
        group, size, _ = _tp()
        if size == 1:
            return x
        x = x.contiguous()
        out = torch.empty((x.shape[0] * size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        group, size, _ = _tp()
        if size == 1:
            return g
        g = g.contiguous()
        out = torch.empty((g.shape[0] // size, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g, group=group)
        return out


class _ReduceScatterRows(torch.autograd.Function):
    """forward: reduce-scatter along dim 0; backward: all-gather along dim 0."""

    @staticmethod
    def forward(ctx, x):
        group, size, _ = _tp()
        if size == 1:
            return x
        x = x.contiguous()
        out = torch.empty((x.shape[0] // size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        group, size, _ = _tp()
        if size == 1:
            return g
        g = g.contiguous()
        out = torch.empty((g.shape[0] * size, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g, group=group)
        return out


# ------------------------------------------------------------------ sequence-parallel region
# Inside the region the activations between the TP seams are sharded by rows (tokens): what enters a column-parallel
# layer was produced by ``gather_rows`` (whose backward is the reduce-scatter that sums the ranks' input gradients), so
# ``copy_to_tp`` has nothing left to do, and what leaves a row-parallel layer is reduce-scattered instead of
# all-reduced.  The layers themselves are unchanged; the decoder layer opens the region (also when it is recomputed
# under activation checkpointing).  Counterpart of the context variable in
# ``areno/engine/parallel/collectives.py:32-49``; the reduce-scatter here is a real one.
_SP_ACTIVE = False


@contextlib.contextmanager
def sequence_parallel_region(enabled: bool = True):
    global _SP_ACTIVE
    prev = _SP_ACTIVE
    _SP_ACTIVE = bool(enabled) and get_context().tp_size > 1
    try:
        yield
    finally:
        _SP_ACTIVE = prev


def in_sequence_parallel() -> bool:
    return _SP_ACTIVE


class _GatherRowsSameGrad(torch.autograd.Function):
    """forward: all-gather along dim 0; backward: this rank's rows of the gradient.  For a consumer that already
    leaves the same, complete gradient on every rank (the LM-head log-prob op sums it over the vocabulary shards)."""

    @staticmethod
    def forward(ctx, x):
        group, size, _ = _tp()
        x = x.contiguous()
        out = torch.empty((x.shape[0] * size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        _, size, rank = _tp()
        n = g.shape[0] // size
        return g[rank * n:(rank + 1) * n].contiguous()


class _LocalRows(torch.autograd.Function):
    """forward: this rank's rows of a replicated tensor; backward: those rows, zeros elsewhere (the producer's own
    backward sums the ranks' contributions)."""

    @staticmethod
    def forward(ctx, x):
        _, size, rank = _tp()
        n = x.shape[0] // size
        ctx.shape = x.shape
        return x[rank * n:(rank + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        _, size, rank = _tp()
        out = g.new_zeros(ctx.shape)
        n = ctx.shape[0] // size
        out[rank * n:(rank + 1) * n] = g
        return out


def reduce_from_tp(x):
    if get_context().tp_size <= 1:
        return x
    if _SP_ACTIVE:
        return _ReduceScatterRows.apply(x)
    return _ReduceFromTP.apply(x)


def copy_to_tp(x):
    if get_context().tp_size <= 1 or _SP_ACTIVE:
        return x
    return _CopyToTP.apply(x)


def gather_rows_same_grad(x):
    return _GatherRowsSameGrad.apply(x) if get_context().tp_size > 1 else x


def local_rows(x):
    """Inside a sequence-parallel region: this rank's rows of a tensor every rank computed in full; else ``x``."""
    return _LocalRows.apply(x) if _SP_ACTIVE else x


def gather_rows(x):
    return _GatherRows.apply(x) if get_context().tp_size > 1 else x


def reduce_scatter_rows(x):
    return _ReduceScatterRows.apply(x) if get_context().tp_size > 1 else x


def all_gather_last_dim(x):
    group, size, _ = _tp()
    if size == 1:
        return x
    x = x.contiguous()
    parts = [torch.empty_like(x) for _ in range(size)]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=-1)
