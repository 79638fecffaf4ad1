"""Mixture-of-experts ops: routers, the device-side route plan, permute / combine and the grouped
expert GEMMs (forward, input gradient, weight gradient), each with a PyTorch fp32 reference used on
CPU and as the test oracle.

Nothing here reads a count back to the host: buffers are sized from the static bound
``routes + experts * 127`` rounded to the 128-row GEMM tile, and the plan tells the grouped GEMM which
tiles are live.  The reference synchronises the host once per MoE layer to get per-expert offsets
(``areno/accel/csrc/moe_permute.cu:280-290``, ``linear.cu:319``) and loops over experts with one
cuBLAS call each; here one persistent tcgen05 launch covers all experts.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib

TILE = 128

_lib.register_signature("areno_topk_softmax_fwd", "piliiippp")
_lib.register_signature("areno_topk_softmax_bwd", "pipppliiipp")
_lib.register_signature("areno_grouped_sigmoid_topk", "ppliiiiifppp")
_lib.register_signature("areno_moe_align", "pliilpppppp")
_lib.register_signature("areno_moe_align_par", "pliilpppppppp")
# from this many routes on the plan is built by the three-launch kernels (one warp per 512 routes) instead of the
# single-CTA kernel, whose time grows with routes x experts (a decode step of 64 sequences x 8 routes over 128
# experts already spends tens of microseconds there)
PAR_ALIGN_MIN_ROUTES = 128


def align_scratch(routes: int, e_count: int, device) -> torch.Tensor:
    return torch.empty(((routes + 511) // 512 + 1) * e_count, dtype=torch.int32, device=device)
_lib.register_signature("areno_moe_permute", "ppilipp")
_lib.register_signature("areno_moe_combine", "pppliipp")
_lib.register_signature("areno_moe_combine_bwd", "ppppillippp")
_lib.register_signature("areno_grouped_gemm_bf16", "pppiiiiippp")
_lib.register_signature("areno_grouped_wgrad_bf16", "pppiiiipipp")


# ------------------------------------------------------------------------------ routers
def topk_softmax_reference(logits, k: int, renorm: bool):
    probs = torch.softmax(logits.float(), -1)
    w, ids = probs.topk(k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return w, ids.to(torch.int32)


class _TopkSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, renorm):
        t, e = logits.shape
        w = torch.empty((t, k), dtype=torch.float32, device=logits.device)
        ids = torch.empty((t, k), dtype=torch.int32, device=logits.device)
        _lib.call("areno_topk_softmax_fwd", logits.data_ptr(), int(logits.dtype == torch.bfloat16), t, e, k, int(renorm),
                  w.data_ptr(), ids.data_ptr(), _lib.stream())
        ctx.save_for_backward(logits, ids, w)
        ctx.args = (k, renorm)
        ctx.mark_non_differentiable(ids)
        return w, ids

    @staticmethod
    def backward(ctx, dw, _dids):
        logits, ids, w = ctx.saved_tensors
        k, renorm = ctx.args
        t, e = logits.shape
        dl = torch.empty((t, e), dtype=torch.float32, device=logits.device)
        _lib.call("areno_topk_softmax_bwd", logits.data_ptr(), int(logits.dtype == torch.bfloat16), ids.data_ptr(),
                  w.data_ptr(), dw.contiguous().float().data_ptr(), t, e, k, int(renorm), dl.data_ptr(), _lib.stream())
        return dl.to(logits.dtype), None, None


def topk_softmax(logits: torch.Tensor, k: int, renorm: bool = True):
    """``softmax -> top-k -> (optional) renormalise``; returns ``(weights fp32 [T,k], ids int32 [T,k])``."""
    if not logits.is_cuda:
        return topk_softmax_reference(logits, k, renorm)
    assert logits.dtype in (torch.float32, torch.bfloat16)
    return _TopkSoftmax.apply(logits.contiguous(), int(k), bool(renorm))


def grouped_sigmoid_topk_reference(logits, bias, n_group, topk_group, k, renorm, scale):
    scores = torch.sigmoid(logits.float())
    choice = scores + (bias.float() if bias is not None else 0.0)
    t, e = scores.shape
    grouped = choice.view(t, n_group, e // n_group)
    gscore = grouped.topk(min(2, e // n_group), dim=-1).values.sum(-1)
    keep = torch.zeros_like(gscore, dtype=torch.bool).scatter(1, gscore.topk(topk_group, dim=-1).indices, True)
    masked = choice.masked_fill(~keep[:, :, None].expand(-1, -1, e // n_group).reshape(t, e), float("-inf"))
    ids = masked.topk(k, dim=-1).indices
    w = scores.gather(1, ids)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scale, ids.to(torch.int32)


def grouped_sigmoid_topk(logits, bias, n_group: int, topk_group: int, k: int, renorm: bool = True, scale: float = 1.0):
    """Sigmoid scores with a selection bias and group-limited top-k (no gradient through the selection;
    weights are returned detached: the caller re-gathers differentiable scores if it trains the gate)."""
    if not logits.is_cuda:
        return grouped_sigmoid_topk_reference(logits, bias, n_group, topk_group, k, renorm, scale)
    t, e = logits.shape
    lg = logits.detach().float().contiguous()
    w = torch.empty((t, k), dtype=torch.float32, device=logits.device)
    ids = torch.empty((t, k), dtype=torch.int32, device=logits.device)
    _lib.call("areno_grouped_sigmoid_topk", lg.data_ptr(), _lib.ptr(bias.float().contiguous() if bias is not None else None),
              t, e, n_group, topk_group, k, int(renorm), float(scale), w.data_ptr(), ids.data_ptr(), _lib.stream())
    return w, ids


# --------------------------------------------------------------------------------- plan
@dataclass
class MoePlan:
    tokens: int
    k: int
    e_count: int
    max_rows: int
    expert_rows: torch.Tensor  # int32 [2 * e_count]: (offset, padded count)
    tile_expert: torch.Tensor  # int32 [max_rows / 128]
    row_route: torch.Tensor    # int32 [max_rows]
    route_row: torch.Tensor    # int32 [tokens * k]
    counts: torch.Tensor       # int32 [e_count] unpadded rows per expert


def max_rows_for(routes: int, experts: int) -> int:
    return (routes + experts * (TILE - 1) + TILE - 1) // TILE * TILE


def align(ids: torch.Tensor, e_lo: int, e_count: int) -> MoePlan:
    """Sort the ``(token, slot)`` routes by expert and pad every expert to whole 128-row tiles."""
    t, k = ids.shape
    routes = t * k
    max_rows = max_rows_for(routes, e_count)
    dev = ids.device
    flat = ids.reshape(-1).to(torch.int32).contiguous()
    if not ids.is_cuda:
        return _align_reference(flat, t, k, e_lo, e_count, max_rows)
    er = torch.empty(2 * e_count, dtype=torch.int32, device=dev)
    te = torch.empty(max_rows // TILE, dtype=torch.int32, device=dev)
    rr = torch.empty(max_rows, dtype=torch.int32, device=dev)
    ro = torch.empty(routes, dtype=torch.int32, device=dev)
    cnt = torch.empty(e_count, dtype=torch.int32, device=dev)
    if routes >= PAR_ALIGN_MIN_ROUTES:
        scratch = align_scratch(routes, e_count, dev)
        _lib.call("areno_moe_align_par", flat.data_ptr(), routes, e_lo, e_count, max_rows, er.data_ptr(), te.data_ptr(),
                  rr.data_ptr(), ro.data_ptr(), cnt.data_ptr(), None, scratch.data_ptr(), _lib.stream())
    else:
        _lib.call("areno_moe_align", flat.data_ptr(), routes, e_lo, e_count, max_rows, er.data_ptr(), te.data_ptr(),
                  rr.data_ptr(), ro.data_ptr(), cnt.data_ptr(), _lib.stream())
    if _lib.BOUNDS_CHECK:     # the plan drives every later gather / scatter and the grouped GEMM: validate it once here
        _lib.check_index("moe plan row_route", rr, routes, low=-1)
        _lib.check_index("moe plan route_row", ro, max_rows, low=-1)
        _lib.check_index("moe plan tile_expert", te, e_count, low=-1)
        _lib.check_index("moe plan expert offsets", er[0::2] + er[1::2], max_rows + 1)
    return MoePlan(t, k, e_count, max_rows, er, te, rr, ro, cnt)


def _align_reference(flat, t, k, e_lo, e_count, max_rows) -> MoePlan:
    er = torch.zeros(2 * e_count, dtype=torch.int32)
    te = torch.full((max_rows // TILE,), -1, dtype=torch.int32)
    rr = torch.full((max_rows,), -1, dtype=torch.int32)
    ro = torch.full((t * k,), -1, dtype=torch.int32)
    cnt = torch.zeros(e_count, dtype=torch.int32)
    off = 0
    for e in range(e_count):
        idx = (flat == e_lo + e).nonzero().flatten()
        n = int(idx.numel())
        padded = (n + TILE - 1) // TILE * TILE
        er[2 * e], er[2 * e + 1], cnt[e] = off, padded, n
        rr[off:off + n] = idx.to(torch.int32)
        ro[idx] = torch.arange(off, off + n, dtype=torch.int32)
        te[off // TILE:(off + padded) // TILE] = e
        off += padded
    return MoePlan(t, k, e_count, max_rows, er, te, rr, ro, cnt)


# ---------------------------------------------------------------------- permute / combine
def _gather_rows_reference(x, plan: MoePlan):
    rr = plan.row_route.long()
    out = torch.zeros((plan.max_rows, x.shape[1]), dtype=x.dtype, device=x.device)
    valid = rr >= 0
    out[valid] = x[rr[valid] // plan.k]
    return out


def _combine_reference(ys, plan: MoePlan, weights):
    ro = plan.route_row.long().view(plan.tokens, plan.k)
    valid = ro >= 0
    rows = ys.float()[ro.clamp(min=0)]                     # [T, k, H]
    w = weights.float() if weights is not None else torch.ones_like(ro, dtype=torch.float32)
    return (rows * (w * valid)[:, :, None]).sum(1).to(ys.dtype)


class _Permute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan: MoePlan):
        ctx.plan = plan
        xs = torch.empty((plan.max_rows, x.shape[1]), dtype=x.dtype, device=x.device)
        _lib.call("areno_moe_permute", x.data_ptr(), plan.row_route.data_ptr(), plan.k, plan.max_rows, x.shape[1],
                  xs.data_ptr(), _lib.stream())
        return xs

    @staticmethod
    def backward(ctx, dxs):
        plan = ctx.plan
        dx = torch.empty((plan.tokens, dxs.shape[1]), dtype=dxs.dtype, device=dxs.device)
        _lib.call("areno_moe_combine", dxs.contiguous().data_ptr(), plan.route_row.data_ptr(), None, plan.tokens, plan.k,
                  dxs.shape[1], dx.data_ptr(), _lib.stream())
        return dx, None


_lib.register_signature("areno_moe_permute_rows", "ppilipp")
_lib.register_signature("areno_router_logits", "ppplii" + "p")
# inference: the largest token count for which the router's logits come from the small fp32 kernel
ROUTER_KERNEL_MAX_TOKENS = 256


def inference_rows_only(*tensors) -> bool:
    """True when no gradient will flow through the MoE ops of this call: padding rows of the expert-sorted buffers
    may then stay uninitialised (a GEMM row only feeds its own output row and nobody gathers a padding row), which
    turns the per-layer work of a decode step from one tile per expert into the routed rows themselves."""
    del tensors      # decided by the autograd mode alone: any grad-enabled pass (training, recompute) fills the padding
    return not torch.is_grad_enabled()


def permute(x: torch.Tensor, plan: MoePlan) -> torch.Tensor:
    """``[T, H] -> [max_rows, H]`` in expert-sorted order (padding rows are zero; unspecified at inference)."""
    if not x.is_cuda:
        return _gather_rows_reference(x, plan)
    if inference_rows_only(x):
        x = x.contiguous()
        xs = torch.empty((plan.max_rows, x.shape[1]), dtype=x.dtype, device=x.device)
        _lib.call("areno_moe_permute_rows", x.data_ptr(), plan.row_route.data_ptr(), plan.k, plan.max_rows, x.shape[1],
                  xs.data_ptr(), _lib.stream())
        return xs
    return _Permute.apply(x.contiguous(), plan)


def router_logits(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight^T`` in fp32 (``weight`` fp32 ``[E, H]``).  A few tokens without gradient take a small kernel
    of this library instead of a cast + library SGEMM."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.float32 and x.dim() == 2
            and 0 < x.shape[0] <= ROUTER_KERNEL_MAX_TOKENS and x.shape[1] % 4 == 0 and x.shape[1] <= 12288
            and inference_rows_only(x, weight)):
        x = x.contiguous()
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        _lib.call("areno_router_logits", x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1],
                  weight.shape[0], _lib.stream())
        return out
    return torch.nn.functional.linear(x.float(), weight)


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ys, weights, plan: MoePlan):
        ctx.plan = plan
        ctx.save_for_backward(ys, weights)
        out = torch.empty((plan.tokens, ys.shape[1]), dtype=ys.dtype, device=ys.device)
        _lib.call("areno_moe_combine", ys.data_ptr(), plan.route_row.data_ptr(), weights.data_ptr(), plan.tokens, plan.k,
                  ys.shape[1], out.data_ptr(), _lib.stream())
        return out

    @staticmethod
    def backward(ctx, dout):
        plan = ctx.plan
        ys, weights = ctx.saved_tensors
        dys = torch.empty_like(ys)
        dw = torch.empty((plan.tokens, plan.k), dtype=torch.float32, device=ys.device)
        _lib.call("areno_moe_combine_bwd", dout.contiguous().data_ptr(), ys.data_ptr(), plan.row_route.data_ptr(),
                  weights.data_ptr(), plan.k, plan.max_rows, plan.tokens * plan.k, ys.shape[1], dys.data_ptr(),
                  dw.data_ptr(), _lib.stream())
        return dys, dw, None


def combine(ys: torch.Tensor, plan: MoePlan, weights: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * ys[row of route (t, j)]`` (routes to non-local experts add 0)."""
    if not ys.is_cuda:
        return _combine_reference(ys, plan, weights)
    return _Combine.apply(ys.contiguous(), weights.float().contiguous(), plan)


# ------------------------------------------------------------------------ grouped GEMMs
def grouped_linear_reference(xs, w, plan: MoePlan):
    out = torch.zeros((plan.max_rows, w.shape[1]), dtype=xs.dtype, device=xs.device)
    if torch.is_grad_enabled() and (xs.requires_grad or w.requires_grad):
        # stay on the autograd graph even when no local expert received a row: under tensor parallelism every
        # rank must run the same backward collectives, whatever the routing gave it
        out = out + (xs.sum() * 0 + w.sum() * 0).to(out.dtype)
    er = plan.expert_rows.tolist()
    for e in range(plan.e_count):
        lo, n = er[2 * e], er[2 * e + 1]
        if n:
            out[lo:lo + n] = (xs[lo:lo + n].float() @ w[e].float().t()).to(xs.dtype)
    return out


def _grouped_gemm(a, b, n, k, e, b_mn, plan: MoePlan):
    out = torch.empty((plan.max_rows, n), dtype=torch.bfloat16, device=a.device)
    _lib.call("areno_grouped_gemm_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), plan.max_rows, n, k, e, int(b_mn),
              plan.tile_expert.data_ptr(), _lib.status_buffer(a.device).data_ptr(), _lib.stream())
    return out


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xs, w, plan: MoePlan):
        e, n, k = w.shape
        ctx.plan = plan
        ctx.save_for_backward(xs, w)
        return _grouped_gemm(xs, w, n, k, e, False, plan)

    @staticmethod
    def backward(ctx, dys):
        plan = ctx.plan
        xs, w = ctx.saved_tensors
        e, n, k = w.shape
        dys = dys.contiguous()
        dxs = None
        if ctx.needs_input_grad[0]:
            # dxs[P, K] = dys[P, N] @ W_e[N, K]: B read as [E, N(reduction), K(output)] rows-major
            dxs = _grouped_gemm(dys, w, k, n, e, True, plan)
        dw = None
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            if main is not None:
                target, acc = main, 1
                w.grad_added_to_main_grad = True
            else:
                target, acc = torch.empty((e, n, k), dtype=torch.bfloat16, device=w.device), 0
            _lib.call("areno_grouped_wgrad_bf16", dys.data_ptr(), xs.data_ptr(), target.data_ptr(), plan.max_rows, n, k, e,
                      plan.expert_rows.data_ptr(), acc, _lib.status_buffer(w.device).data_ptr(), _lib.stream())
            dw = None if acc else target
        return dxs, dw, None


def grouped_linear(xs: torch.Tensor, w: torch.Tensor, plan: MoePlan) -> torch.Tensor:
    """Rows of ``xs [max_rows, K]`` times their expert's ``w[e] [N, K]`` transposed -> ``[max_rows, N]``.
    Rows of unused tiles are left unspecified (nothing downstream reads them)."""
    if not xs.is_cuda:
        return grouped_linear_reference(xs, w, plan)
    assert xs.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous()
    return _GroupedLinear.apply(xs.contiguous(), w, plan)
