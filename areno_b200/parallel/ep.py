"""Expert parallelism over peer memory: the all-to-all that takes every token to the ranks owning its experts
and brings the expert outputs back (``csrc/ep.cu``), wrapped as two differentiable ops.

Layout: the ranks of ``group`` each own ``E / n`` consecutive experts and their own tokens (the group is the
data-parallel group of the job).  ``EpComm`` keeps, in a symmetric heap (``parallel/symm.py``), two slots of

* ``pub``      bf16 ``[cap * k, H]``: rows this rank publishes for its peers to pull (tokens on the way out,
  gradients of the combined rows on the way back);
* ``inbox``    bf16 ``[cap * k, H]``: one row per (token, slot) of this rank, stored there by the expert owners;
* ``ids_all``  int32 ``[n, cap * k]``: the routing tables of all ranks (every rank stores its own into everybody's).

``dispatch(x, ids)`` returns the expert-sorted rows that hit the local experts plus the plan;
``combine(ys, weights, plan)`` returns the weighted sum per local token.  Their backward passes are each other's
data movement with the roles swapped, so training works through ordinary autograd:

    rows, plan = ep.dispatch(x, ids)                 # publish -> barrier -> align -> pull
    rows = grouped_linear(...act(grouped_linear(rows, w_gate_up, plan))..., w_down, plan)
    out = ep.combine(rows, weights, plan)            # push -> barrier -> weighted sum

Every rank of the group must make the same sequence of calls with the same ``cap`` (the row counts themselves may
differ and stay on the device).  The expert-sorted buffer is sized for ``capacity`` times the mean load; routes
beyond it are dropped by the plan and counted (``EpComm.dropped()``), which callers treat as an error unless they
opted into token dropping.  Waits inside the barrier kernel are bounded and report through the status word.

The reference has no counterpart: it shards experts over TP, replicates the tokens and all-reduces
(``areno/models/qwen3/model.py:99-116``).
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from ..ops import _lib
from ..ops import moe as moe_ops
from .symm import SymmHeap, TpDesc, _as_tensor, _Blob, _ptr_array

_lib.register_signature("areno_ep_publish_ids", "iippllp")
_lib.register_signature("areno_ep_pull_rows", "ipplii" + "plip")
_lib.register_signature("areno_ep_push_rows", "ippl" + "plip")
_lib.register_signature("areno_moe_align_capped", "pliilppppppp")


@dataclass
class EpPlan:
    """Routing plan of one MoE call on this rank: ``moe`` sorts the routes of all ranks that hit a local expert;
    ``slot`` is the heap slot the call's buffers live in."""

    moe: moe_ops.MoePlan
    slot: int
    tokens: int
    k: int


class EpComm:
    HEADER = 4096

    def __init__(self, group, size: int, rank: int, hidden: int, cap_tokens: int, k: int, num_experts: int,
                 device: torch.device, capacity: float = 2.0):
        if hidden % 8 != 0 or num_experts % size != 0:
            raise ValueError("hidden must be a multiple of 8 and num_experts a multiple of the group size")
        self.group, self.n, self.rank, self.device = group, int(size), int(rank), device
        self.hidden, self.cap, self.k = int(hidden), int(cap_tokens), int(k)
        self.e_local = num_experts // self.n
        self.e_lo = self.rank * self.e_local
        self.cap_routes = self.cap * self.k
        # rows of the expert-sorted buffer: `capacity` times the mean number of routes per rank, never less than a
        # tile per expert and never more than the static bound that covers every routing
        mean = self.cap_routes
        bound = moe_ops.max_rows_for(self.n * self.cap_routes, self.e_local)
        want = int(capacity * mean) + self.e_local * moe_ops.TILE
        self.max_rows = min(bound, (want + moe_ops.TILE - 1) // moe_ops.TILE * moe_ops.TILE)
        row_bytes = self.cap_routes * self.hidden * 2
        self.row_bytes = (row_bytes + 4095) // 4096 * 4096
        self.ids_bytes = (self.n * self.cap_routes * 4 + 4095) // 4096 * 4096
        self.slot_bytes = 2 * self.row_bytes + self.ids_bytes
        total = self.HEADER + 2 * self.slot_bytes
        self.heap = SymmHeap(group, self.n, self.rank, total, device, multicast=False)
        self.status = _lib.status_buffer(device)
        self.wait_ms = int(os.environ.get("ARENO_EP_WAIT_MS", "20000"))
        bases = self.heap.bases
        self._flag_array = _ptr_array(bases)
        self._desc = TpDesc(self.n, self.rank, self._flag_array, None, None, None, None, None, None,
                            self.status.data_ptr(), self.wait_ms)
        self._pub, self._inbox, self._ids, self._ptrs = [], [], [], []
        local = self.heap.local_base
        for s in range(2):
            off = self.HEADER + s * self.slot_bytes
            self._pub.append(_as_tensor(local + off, self.cap_routes * self.hidden, device).view(self.cap_routes, self.hidden))
            self._inbox.append(_as_tensor(local + off + self.row_bytes, self.cap_routes * self.hidden, device)
                               .view(self.cap_routes, self.hidden))
            ids = torch.as_tensor(_Blob(local + off + 2 * self.row_bytes, self.n * self.cap_routes, "<i4"), device=device)
            self._ids.append(ids.view(self.n, self.cap_routes))
            self._ptrs.append({"pub": _ptr_array([b + off for b in bases]),
                               "inbox": _ptr_array([b + off + self.row_bytes for b in bases]),
                               "ids": _ptr_array([b + off + 2 * self.row_bytes for b in bases])})
        self._route_index = torch.arange(self.cap_routes, dtype=torch.int32, device=device)    # see _identity
        self._dropped = torch.zeros(1, dtype=torch.int32, device=device)
        self._dropped_total = torch.zeros(1, dtype=torch.int64, device=device)
        self.calls = 0

    # ------------------------------------------------------------------------------ pieces
    def _next_slot(self) -> int:
        s = self.calls & 1
        self.calls += 1
        return s

    def barrier(self) -> None:
        _lib.call("areno_tp_barrier", ctypes.addressof(self._desc), _lib.stream())

    def dropped(self) -> int:
        """Routes dropped so far because an expert-sorted buffer was full (synchronising read)."""
        return int(self._dropped_total.item())

    def _plan(self, slot: int, tokens: int) -> EpPlan:
        ids_all = self._ids[slot]
        routes = self.n * self.cap_routes
        dev = self.device
        er = torch.empty(2 * self.e_local, dtype=torch.int32, device=dev)
        te = torch.empty(self.max_rows // moe_ops.TILE, dtype=torch.int32, device=dev)
        rr = torch.empty(self.max_rows, dtype=torch.int32, device=dev)
        ro = torch.empty(routes, dtype=torch.int32, device=dev)
        cnt = torch.empty(self.e_local, dtype=torch.int32, device=dev)
        if routes >= moe_ops.PAR_ALIGN_MIN_ROUTES:
            scratch = moe_ops.align_scratch(routes, self.e_local, dev)
            _lib.call("areno_moe_align_par", ids_all.data_ptr(), routes, self.e_lo, self.e_local, self.max_rows,
                      er.data_ptr(), te.data_ptr(), rr.data_ptr(), ro.data_ptr(), cnt.data_ptr(),
                      self._dropped.data_ptr(), scratch.data_ptr(), _lib.stream())
        else:
            _lib.call("areno_moe_align_capped", ids_all.data_ptr(), routes, self.e_lo, self.e_local, self.max_rows,
                      er.data_ptr(), te.data_ptr(), rr.data_ptr(), ro.data_ptr(), cnt.data_ptr(),
                      self._dropped.data_ptr(), _lib.stream())
        self._dropped_total += self._dropped
        plan = moe_ops.MoePlan(self.n * self.cap, self.k, self.e_local, self.max_rows, er, te, rr, ro, cnt)
        return EpPlan(plan, slot, tokens, self.k)

    def _pull(self, slot: int, plan: EpPlan, per_token: bool) -> torch.Tensor:
        rows = torch.empty((self.max_rows, self.hidden), dtype=torch.bfloat16, device=self.device)
        _lib.call("areno_ep_pull_rows", self.n, self._ptrs[slot]["pub"], plan.moe.row_route.data_ptr(), self.cap_routes,
                  self.k, int(per_token), rows.data_ptr(), self.max_rows, self.hidden, _lib.stream())
        return rows

    def _push(self, slot: int, plan: EpPlan, rows: torch.Tensor) -> None:
        rows = rows.contiguous()
        _lib.call("areno_ep_push_rows", self.n, self._ptrs[slot]["inbox"], plan.moe.row_route.data_ptr(), self.cap_routes,
                  rows.data_ptr(), self.max_rows, self.hidden, _lib.stream())

    # --------------------------------------------------------------------------------- ops
    def dispatch(self, x: torch.Tensor, ids: torch.Tensor):
        """``x [T, H]`` bf16, ``ids [T, k]`` int32 global expert ids -> (expert-sorted rows ``[max_rows, H]``, plan)."""
        if x.shape[0] > self.cap or x.shape[1] != self.hidden or ids.shape != (x.shape[0], self.k):
            raise ValueError(f"dispatch: x {tuple(x.shape)} / ids {tuple(ids.shape)} do not fit cap={self.cap}, "
                             f"hidden={self.hidden}, k={self.k}")
        slot = self._next_slot()
        t = x.shape[0]
        flat = ids.reshape(-1).to(torch.int32).contiguous()
        _lib.call("areno_ep_publish_ids", self.n, self.rank, self._ptrs[slot]["ids"], flat.data_ptr(), t * self.k,
                  self.cap_routes, _lib.stream())
        plan_holder: list = []
        rows = _Dispatch.apply(x, self, slot, plan_holder)
        return rows, plan_holder[0]

    def combine(self, ys: torch.Tensor, weights: torch.Tensor, plan: EpPlan) -> torch.Tensor:
        """Expert outputs ``ys [max_rows, H]`` -> ``[T, H]``: ``sum_j weights[t, j] * y(t, j)``."""
        return _Combine.apply(ys, weights, self, plan)

    def close(self) -> None:
        self.heap.close()


def _identity(routes: int, device, comm=None) -> torch.Tensor:
    """Route map in which route (t, j) lives in row t * k + j: lets the local combine kernels run on an inbox."""
    if comm is not None and routes <= comm.cap_routes:
        return comm._route_index[:routes]
    return torch.arange(routes, dtype=torch.int32, device=device)


def _weighted_sum(rows: torch.Tensor, weights: torch.Tensor | None, tokens: int, k: int, comm=None) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * rows[t * k + j]`` (plain sum without weights)."""
    out = torch.empty((tokens, rows.shape[1]), dtype=rows.dtype, device=rows.device)
    _lib.call("areno_moe_combine", rows.data_ptr(), _identity(tokens * k, rows.device, comm).data_ptr(), _lib.ptr(weights),
              tokens, k, rows.shape[1], out.data_ptr(), _lib.stream())
    return out


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm: EpComm, slot: int, plan_holder: list):
        t = x.shape[0]
        comm._pub[slot][:t].copy_(x)                 # tokens on the way out: one row per token
        comm.barrier()                               # every rank's tokens and routing tables are in place
        plan = comm._plan(slot, t)
        rows = comm._pull(slot, plan, per_token=True)
        plan_holder.append(plan)
        ctx.comm, ctx.plan = comm, plan
        return rows

    @staticmethod
    def backward(ctx, d_rows):
        comm, plan = ctx.comm, ctx.plan
        slot = comm._next_slot()
        comm._push(slot, plan, d_rows)               # gradient of a pull is a push to the rows' owners
        comm.barrier()
        t, k = plan.tokens, plan.k
        dx = _weighted_sum(comm._inbox[slot][: t * k], None, t, k, comm)      # sum over the k routes of a token
        return dx, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ys, weights, comm: EpComm, plan: EpPlan):
        comm._push(plan.slot, plan, ys)              # every output row to the rank that owns its token
        comm.barrier()
        t, k = plan.tokens, plan.k
        inbox = comm._inbox[plan.slot][: t * k]
        weights = weights.float().contiguous()
        out = _weighted_sum(inbox, weights, t, k, comm)
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            ctx.save_for_backward(inbox.clone(), weights)   # the slot is reused two calls later
        ctx.comm, ctx.plan = comm, plan
        return out

    @staticmethod
    def backward(ctx, dout):
        comm, plan = ctx.comm, ctx.plan
        rows_in, weights = ctx.saved_tensors
        t, k = plan.tokens, plan.k
        d_rows_local = torch.empty_like(rows_in)
        dweights = torch.empty((t, k), dtype=torch.float32, device=dout.device)
        _lib.call("areno_moe_combine_bwd", dout.contiguous().data_ptr(), rows_in.data_ptr(),
                  _identity(t * k, dout.device, comm).data_ptr(), weights.data_ptr(), k, t * k, t * k, rows_in.shape[1],
                  d_rows_local.data_ptr(), dweights.data_ptr(), _lib.stream())
        slot = comm._next_slot()
        comm._pub[slot][: t * k].copy_(d_rows_local)         # one row per route, for the expert owners to pull
        comm.barrier()
        d_ys = comm._pull(slot, plan, per_token=False)
        comm.barrier()       # the pulls are done before anybody republishes (the next call may come at once)
        return d_ys, dweights, None, None


# ------------------------------------------------------------------------------------------------------------
# Collective fallback and the per-model runtime
# ------------------------------------------------------------------------------------------------------------
class _GroupGatherRows(torch.autograd.Function):
    """All-gather along dim 0 over ``group``; the backward is the matching reduce-scatter (sum)."""

    @staticmethod
    def forward(ctx, x, group, size):
        ctx.group, ctx.size = group, size
        x = x.contiguous()
        out = torch.empty((x.shape[0] * size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        torch.distributed.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = torch.empty((g.shape[0] // ctx.size, *g.shape[1:]), dtype=g.dtype, device=g.device)
        torch.distributed.reduce_scatter_tensor(out, g, group=ctx.group)
        return out, None, None


class _GroupReduceScatterRows(torch.autograd.Function):
    """Reduce-scatter (sum) along dim 0 over ``group``; the backward is the matching all-gather."""

    @staticmethod
    def forward(ctx, x, group, size):
        ctx.group, ctx.size = group, size
        x = x.contiguous()
        out = torch.empty((x.shape[0] // size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        torch.distributed.reduce_scatter_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = torch.empty((g.shape[0] * ctx.size, *g.shape[1:]), dtype=g.dtype, device=g.device)
        torch.distributed.all_gather_into_tensor(out, g, group=ctx.group)
        return out, None, None


def _reduce_scatter_any(x, group, size):
    """``reduce_scatter_tensor`` where the backend has it, all-reduce + slice otherwise (gloo)."""
    if x.is_cuda:
        return _GroupReduceScatterRows.apply(x, group, size)
    return _ReduceScatterViaAllReduce.apply(x, group, size)


def _gather_any(x, group, size):
    if x.is_cuda:
        return _GroupGatherRows.apply(x, group, size)
    return _GatherViaAllGather.apply(x, group, size)


class _GatherViaAllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, size):
        ctx.group, ctx.size = group, size
        ctx.rank = torch.distributed.get_rank(group)
        parts = [torch.empty_like(x) for _ in range(size)]
        torch.distributed.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        torch.distributed.all_reduce(g, group=ctx.group)
        n = g.shape[0] // ctx.size
        return g[ctx.rank * n:(ctx.rank + 1) * n], None, None


class _ReduceScatterViaAllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, size):
        ctx.group, ctx.size = group, size
        ctx.rank = torch.distributed.get_rank(group)
        x = x.contiguous().clone()
        torch.distributed.all_reduce(x, group=group)
        n = x.shape[0] // size
        return x[ctx.rank * n:(ctx.rank + 1) * n].clone()

    @staticmethod
    def backward(ctx, g):
        parts = [torch.empty_like(g) for _ in range(ctx.size)]
        torch.distributed.all_gather(parts, g.contiguous(), group=ctx.group)
        return torch.cat(parts, dim=0), None, None


class EpCommCollective:
    """Expert parallelism on library collectives: tokens, routing tables and routing weights are all-gathered
    (padded to ``cap`` rows per rank), every rank serves the routes that hit its experts, and the partial outputs
    are reduce-scattered back to the tokens' owners.  Same interface as ``EpComm``; it is the baseline the
    peer-memory path is measured against, the path CPU (gloo) runs take, and differentiable through the
    collectives' own backward rules."""

    kind = "collective"

    def __init__(self, group, size: int, rank: int, hidden: int, cap_tokens: int, k: int, num_experts: int, device):
        self.group, self.n, self.rank, self.device = group, int(size), int(rank), device
        self.hidden, self.cap, self.k = int(hidden), int(cap_tokens), int(k)
        self.e_local = num_experts // self.n
        self.e_lo = self.rank * self.e_local

    def dispatch(self, x: torch.Tensor, ids: torch.Tensor):
        t = x.shape[0]
        if t > self.cap:
            raise ValueError(f"dispatch: {t} tokens do not fit cap={self.cap}")
        pad = self.cap - t
        xp = torch.nn.functional.pad(x, (0, 0, 0, pad)) if pad else x
        idp = torch.nn.functional.pad(ids.to(torch.int32), (0, 0, 0, pad), value=-1) if pad else ids.to(torch.int32)
        x_all = _gather_any(xp, self.group, self.n)
        ids_all = _gather_any(idp.contiguous(), self.group, self.n)
        plan = moe_ops.align(ids_all, self.e_lo, self.e_local)
        rows = moe_ops.permute(x_all, plan)
        return rows, EpPlan(plan, 0, t, self.k)

    def combine(self, ys: torch.Tensor, weights: torch.Tensor, plan: EpPlan) -> torch.Tensor:
        t = plan.tokens
        pad = self.cap - t
        wp = torch.nn.functional.pad(weights.float(), (0, 0, 0, pad)) if pad else weights.float()
        w_all = _gather_any(wp.contiguous(), self.group, self.n)
        partial = moe_ops.combine(ys, plan.moe, w_all)              # [n * cap, H]: this rank's experts only
        mine = _reduce_scatter_any(partial, self.group, self.n)     # [cap, H]
        return mine[:t]

    def dropped(self) -> int:
        return 0

    def barrier(self) -> None:
        torch.distributed.barrier(group=self.group)

    def close(self) -> None:
        pass


class EpRuntime:
    """The expert-parallel communicators of one process.  A communicator is sized for a token capacity; forward
    passes of different sizes (a training micro-batch, a prefill chunk, a decode step) use different ones, picked
    by power-of-two bucket.  Every rank of the group must run the same sequence of MoE calls with the same
    bucket, so callers that cannot know the other ranks' sizes agree on them first (``agree_max``) and pin the
    bucket for the pass (``with runtime.pinned(tokens)``)."""

    MIN_CAP = 64

    def __init__(self, ctx, hidden: int, k: int, num_experts: int, device, capacity: float | None = None,
                 impl: str | None = None):
        self.ctx, self.hidden, self.k, self.num_experts = ctx, int(hidden), int(k), int(num_experts)
        self.device = torch.device(device)
        self.capacity = float(capacity if capacity is not None else os.environ.get("ARENO_EP_CAPACITY", "2.0"))
        impl = impl or os.environ.get("ARENO_EP_IMPL", "peer")
        self.impl = impl if self.device.type == "cuda" else "collective"
        self._comms: dict[int, object] = {}
        self._pinned: int | None = None

    @staticmethod
    def bucket(tokens: int) -> int:
        cap = EpRuntime.MIN_CAP
        while cap < tokens:
            cap *= 2
        return cap

    def comm(self, tokens: int):
        cap = self.bucket(self._pinned if self._pinned is not None else tokens)
        if tokens > cap:
            raise ValueError(f"{tokens} tokens exceed the bucket pinned for this pass ({cap})")
        c = self._comms.get(cap)
        if c is None:
            ctx = self.ctx
            if self.impl == "collective":
                c = EpCommCollective(ctx.ep_group, ctx.ep_size, ctx.ep_rank, self.hidden, cap, self.k,
                                     self.num_experts, self.device)
            else:
                c = EpComm(ctx.ep_group, ctx.ep_size, ctx.ep_rank, self.hidden, cap, self.k, self.num_experts,
                           self.device, capacity=self.capacity)
            self._comms[cap] = c
        return c

    def pinned(self, tokens: int):
        """Context manager: every MoE call inside uses the bucket of ``tokens`` (the group-wide maximum)."""
        rt = self

        class _Pin:
            def __enter__(self_inner):
                self_inner.prev = rt._pinned
                rt._pinned = int(tokens)

            def __exit__(self_inner, *exc):
                rt._pinned = self_inner.prev
                return False

        return _Pin()

    def agree_max(self, values: list[int]) -> list[int]:
        """Element-wise maximum of ``values`` over the group, computed on the host (gloo)."""
        t = torch.tensor(list(values), dtype=torch.int64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=self.ctx.ep_ctl_group)
        return [int(v) for v in t.tolist()]

    def dropped(self) -> int:
        return sum(int(c.dropped()) for c in self._comms.values())

    def close(self) -> None:
        for c in self._comms.values():
            c.close()
        self._comms.clear()
