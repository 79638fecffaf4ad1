"""Tensor-parallel building blocks shared by the model families.

Every linear stores its weight ``[out_local, in]`` (row-major, K-major for the tcgen05 GEMM) and
calls ``ops.gemm.linear``.  Column-parallel layers shard the output features, row-parallel layers
shard the input features and reduce over the TP group.  Parameters carry two annotations used by
the trainer and the checkpoint code:

* ``tp_shard``: ``("col" | "row" | "vocab" | "qkv" | "merged" | None, meta)`` describing how the
  local tensor maps onto the full HF tensor(s);
* ``tp_replicated_grad``: the parameter is replicated over TP.  ``True``: each rank holds only the part of the
  gradient that flows through its own heads / experts and the trainer sums them (per-head q / k norms, router
  gates); ``"same"``: every rank already holds the full gradient (norm scales in front of a column-parallel
  layer, biases added after the row-parallel reduce) and nothing is reduced.

Role of ``areno/engine/layers/{linear,vocab,mlp,norm}.py`` in the reference.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import activation, embedding as emb_ops, gemm, norm as norm_ops
from ..parallel import collectives as coll
from ..parallel.context import get_context
from ..parallel.symm import TpPartial, get_tp_comm


def _param(shape, dtype, device) -> nn.Parameter:
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=True)


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float, dtype, device, offset: float = 0.0, with_scale: bool = True):
        super().__init__()
        self.eps = eps
        self.offset = offset
        self.weight = _param((hidden,), dtype, device) if with_scale else None
        if self.weight is not None:
            # default: the norm runs on a replicated activation and feeds a layer that sums the input gradient
            # over TP; owners that apply it to their local heads switch the annotation to True (partial)
            self.weight.tp_replicated_grad = "same"

    def forward(self, x, residual=None, want_sum: bool = False):
        """``want_sum``: for an input that is still spread over the TP group and has no residual (the embedding
        output), also return the reduced input itself, which becomes the residual stream."""
        if isinstance(x, gemm.SplitKPartial):
            # a decode-sized row-parallel GEMM left its split-K partials for us: fold, add, normalise
            y, h = norm_ops.splitk_residual_rmsnorm(x, residual, self.weight, self.eps, self.offset)
            return (y, h) if residual is not None else y
        if isinstance(x, TpPartial):
            # x is a row-parallel partial still spread over the TP group's inboxes: reduce it, add the
            # residual stream and normalise in one kernel
            y, h = x.comm.reduce_rmsnorm(x, residual, self.weight, self.eps, self.offset)
            return (y, h) if (residual is not None or want_sum) else y
        return norm_ops.rmsnorm(x, self.weight, self.eps, residual=residual, w_offset=self.offset)


class ColumnParallelLinear(nn.Module):
    """y_local = x W_localᵀ (+ b_local); input replicated over TP, output sharded on features."""

    def __init__(self, in_features: int, out_features: int, bias: bool, dtype, device, gather_output: bool = False):
        super().__init__()
        ctx = get_context()
        assert out_features % ctx.tp_size == 0, "column-parallel output must divide tp_size"
        self.in_features, self.out_features = in_features, out_features
        self.out_local = out_features // ctx.tp_size
        self.gather_output = gather_output
        self.weight = _param((self.out_local, in_features), dtype, device)
        self.weight.tp_shard = ("col", None)
        self.bias = _param((self.out_local,), dtype, device) if bias else None
        if self.bias is not None:
            self.bias.tp_shard = ("col", None)

    def forward(self, x):
        x = coll.copy_to_tp(x)
        y = gemm.linear(x, self.weight, self.bias)
        if self.gather_output:
            y = coll.all_gather_last_dim(y)
        return y


class MergedColumnParallelLinear(nn.Module):
    """Several column-parallel projections of the same input fused into one GEMM (gate_up)."""

    def __init__(self, in_features: int, out_features: list[int], bias: bool, dtype, device):
        super().__init__()
        ctx = get_context()
        for o in out_features:
            assert o % ctx.tp_size == 0
        self.in_features = in_features
        self.out_features = list(out_features)
        self.out_locals = [o // ctx.tp_size for o in out_features]
        self.weight = _param((sum(self.out_locals), in_features), dtype, device)
        self.weight.tp_shard = ("merged", self.out_locals)
        self.bias = _param((sum(self.out_locals),), dtype, device) if bias else None
        if self.bias is not None:
            self.bias.tp_shard = ("merged", self.out_locals)

    def forward(self, x):
        return gemm.linear(coll.copy_to_tp(x), self.weight, self.bias)


def split_heads(num_heads: int, num_kv_heads: int, tp: int, rank: int) -> tuple[int, int, int, int, int]:
    """Head layout of one TP rank: ``(hq_local, q_lo, q_n, hkv_local, kv_rep)``.

    ``hq_local`` query heads are computed locally, of which the first ``q_n`` are real heads
    ``[q_lo, q_lo + q_n)`` of the model and the rest zero-weight padding.  Padding only occurs when the
    layout is wider than the query heads divide: the ``gq`` query heads of a KV group are then dealt out in
    blocks of ``ceil(gq / kv_rep)`` over the ``kv_rep`` ranks that share the group's KV head."""
    if num_kv_heads >= tp:
        assert num_kv_heads % tp == 0 and num_heads % tp == 0
        hq = num_heads // tp
        return hq, rank * hq, hq, num_kv_heads // tp, 1
    assert tp % num_kv_heads == 0
    rep = tp // num_kv_heads
    if num_heads % tp == 0:
        hq = num_heads // tp
        return hq, rank * hq, hq, 1, rep
    assert num_heads % num_kv_heads == 0
    gq = num_heads // num_kv_heads
    hq = (gq + rep - 1) // rep
    group, j = rank // rep, rank % rep
    lo = min(j * hq, gq)
    n = min((j + 1) * hq, gq) - lo
    return hq, group * gq + lo, n, 1, rep


class QKVParallelLinear(nn.Module):
    """Fused q/k/v projection.  Q heads are split over TP; KV heads are split when they divide
    ``tp_size`` and otherwise replicated (``tp_size`` a multiple of the KV head count).  An
    inference-only layout may carry zero-weight padding heads (see ``split_heads``)."""

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, bias: bool, dtype, device,
                 q_mult: int = 1):
        super().__init__()
        ctx = get_context()
        tp = ctx.tp_size
        self.hq, self.q_lo, self.q_n, self.hkv, self.kv_rep = split_heads(num_heads, num_kv_heads, tp, ctx.tp_rank)
        self.padded = self.q_n != self.hq or num_heads % tp != 0
        self.head_dim = head_dim
        self.q_mult = q_mult  # 2 when the projection also carries an output gate per q head
        out = (self.hq * q_mult + 2 * self.hkv) * head_dim
        self.weight = _param((out, hidden), dtype, device)
        meta = (self.hq * q_mult, self.hkv, head_dim, self.kv_rep)
        if num_heads % tp != 0:
            # uneven layout: (local q rows incl. padding, kv heads, head_dim, kv replication, first real q row of the
            # full tensor, real q rows, q rows of the full tensor), rows in units of heads x q_mult
            meta = meta + (self.q_lo * q_mult, self.q_n * q_mult, num_heads * q_mult)
        self.weight.tp_shard = ("qkv", meta)
        self.bias = _param((out,), dtype, device) if bias else None
        if self.bias is not None:
            self.bias.tp_shard = ("qkv", meta)
        if self.kv_rep > 1:
            # k/v rows are replicated over `kv_rep` ranks: their grads must be summed over replicas
            self.weight.kv_replicated = self.kv_rep
            if self.bias is not None:
                self.bias.kv_replicated = self.kv_rep

    def forward(self, x):
        return gemm.linear(coll.copy_to_tp(x), self.weight, self.bias)


class RowParallelLinear(nn.Module):
    """y = sum_over_tp(x_local W_localᵀ) (+ b); input sharded on features, output replicated."""

    def __init__(self, in_features: int, out_features: int, bias: bool, dtype, device, reduce_output: bool = True,
                 in_range: tuple[int, int, int] | None = None):
        """``in_range = (in_local, lo, n)``: this rank's input has ``in_local`` features of which the first ``n`` are
        features ``[lo, lo + n)`` of the full layer and the rest multiply zero weights (an attention output
        projection behind padded heads)."""
        super().__init__()
        ctx = get_context()
        self.out_features = out_features
        self.reduce_output = reduce_output
        if in_range is not None:
            self.in_local = int(in_range[0])
        else:
            assert in_features % ctx.tp_size == 0
            self.in_local = in_features // ctx.tp_size
        # set by owners whose next op is an RMSNorm with residual: lets inference hand the un-reduced
        # partial to the fused reduce + residual + norm kernel instead of calling an all-reduce
        self.defer_reduce = False
        self.weight = _param((out_features, self.in_local), dtype, device)
        self.weight.tp_shard = ("row", None if in_range is None else (int(in_range[1]), int(in_range[2])))
        self.bias = _param((out_features,), dtype, device) if bias else None
        if self.bias is not None:
            self.bias.tp_replicated_grad = "same"

    def forward(self, x):
        ctx = get_context()
        if ctx.tp_size == 1:
            if (self.defer_reduce and self.bias is None and x.is_cuda and not torch.is_grad_enabled()
                    and x.dim() == 2 and x.shape[0] <= 128 and self.weight.dtype == torch.bfloat16):
                return gemm.gemm_partials(x, self.weight)
            return gemm.linear(x, self.weight, self.bias)
        if self.defer_reduce and self.bias is None and x.is_cuda and not torch.is_grad_enabled():
            comm = get_tp_comm(ctx)
            x2 = x.reshape(-1, x.shape[-1])
            # inference with a peer-memory communicator: leave the partial product in the symmetric heap; the
            # RMSNorm that follows reduces it over the group, adds the residual and normalises in one kernel
            if comm is not None and comm.hidden == self.out_features and 0 < x2.shape[0] <= comm.max_rows:
                return comm.row_linear(x2, self.weight)
        y = gemm.linear(x, self.weight, None)
        if self.reduce_output:
            y = coll.reduce_from_tp(y)
        if self.bias is not None:
            y = y + self.bias
        return y


class VocabParallelEmbedding(nn.Module):
    def __init__(self, vocab: int, hidden: int, dtype, device, scale: float = 1.0):
        super().__init__()
        ctx = get_context()
        self.vocab = vocab
        self.per_rank = (vocab + ctx.tp_size - 1) // ctx.tp_size
        # pad so every rank holds the same number of rows (multiple of 8 keeps 16-byte alignment)
        self.per_rank = (self.per_rank + 7) // 8 * 8
        self.vocab_start = ctx.tp_rank * self.per_rank
        self.scale = scale
        self.weight = _param((self.per_rank, hidden), dtype, device)
        self.weight.tp_shard = ("vocab", vocab)

    def forward(self, ids, defer_reduce: bool = False):
        """``defer_reduce``: the caller's next op is an RMSNorm that can take the un-reduced lookup (rows owned by
        other ranks are zero) and fold the TP sum into its own kernel."""
        ctx = get_context()
        if defer_reduce and ctx.tp_size > 1 and ids.is_cuda and not torch.is_grad_enabled() and ids.dim() == 1:
            comm = get_tp_comm(ctx)
            if comm is not None and comm.hidden == self.weight.shape[1] and 0 < ids.numel() <= comm.max_rows:
                part = comm.new_partial(ids.numel())
                emb_ops.embedding(ids, self.weight, self.vocab_start, self.scale, out=part.local)
                return part
        out = emb_ops.embedding(ids, self.weight, self.vocab_start, self.scale)
        return coll.reduce_from_tp(out)


class VocabParallelLMHead(nn.Module):
    """Output projection onto the local vocabulary shard (weight may be tied to the embedding)."""

    def __init__(self, vocab: int, hidden: int, dtype, device, tied_to: VocabParallelEmbedding | None = None):
        super().__init__()
        ctx = get_context()
        self.vocab = vocab
        per_rank = (vocab + ctx.tp_size - 1) // ctx.tp_size
        self.per_rank = (per_rank + 7) // 8 * 8
        self.vocab_start = ctx.tp_rank * self.per_rank
        self.valid_local = max(0, min(self.per_rank, vocab - self.vocab_start))
        if tied_to is not None:
            self.weight = tied_to.weight
        else:
            self.weight = _param((self.per_rank, hidden), dtype, device)
            self.weight.tp_shard = ("vocab", vocab)

    def forward(self, hidden, out_dtype=torch.bfloat16):
        """Logits over the local shard ``[rows, per_rank]`` (columns past ``valid_local`` are padding)."""
        if hidden.is_cuda and not (torch.is_grad_enabled() and hidden.requires_grad):
            return gemm.gemm(hidden.reshape(-1, hidden.shape[-1]), self.weight, out_dtype=out_dtype)
        return gemm.linear(hidden, self.weight)


class GatedMLP(nn.Module):
    def __init__(self, hidden: int, intermediate: int, act: str, bias: bool, dtype, device):
        super().__init__()
        self.gate_up = MergedColumnParallelLinear(hidden, [intermediate, intermediate], bias, dtype, device)
        self.down = RowParallelLinear(intermediate, hidden, bias, dtype, device)
        self.act = act

    def forward(self, x):
        gup = self.gate_up
        if (x.is_cuda and not torch.is_grad_enabled() and gup.bias is None and gup.out_locals[0] % 8 == 0 and x.dim() == 2
                and x.shape[0] > 128 and x.shape[0] * gup.out_locals[0] >= 148 * 128 * 128):
            # inference on more than one row tile (prefill, scoring): the activation runs in the GEMM epilogue and
            # the pre-activation is never written (14 % faster at 4096 rows).  Decode keeps the separate kernel:
            # with one tile per CTA the extra epilogue work is not hidden behind another tile's main loop, and a
            # batch of a few hundred rows with fewer output tiles than SMs is better served by split-K.
            a = gemm.gated_linear(coll.copy_to_tp(x), gup.weight, self.act)
        else:
            gu = gup(x)
            a = activation.silu_and_mul(gu) if self.act == "silu" else activation.gelu_tanh_and_mul(gu)
        return self.down(a)
