"""MoE kernels against their PyTorch fp32 references on a B200."""

from __future__ import annotations

import pytest
import torch

from areno_b200.ops import _lib, moe as moe_ops

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("tokens,E,k,renorm,dtype", [(513, 128, 8, True, torch.float32), (64, 8, 2, False, torch.float32),
                                                      (300, 60, 4, True, torch.bfloat16), (7, 512, 16, True, torch.float32)])
def test_topk_softmax_fwd_bwd(tokens, E, k, renorm, dtype):
    torch.manual_seed(0)
    logits = (torch.randn(tokens, E, device="cuda") * 2).to(dtype).requires_grad_()
    w, ids = moe_ops.topk_softmax(logits, k, renorm)
    ref_in = logits.detach().float().requires_grad_()
    w_ref, ids_ref = moe_ops.topk_softmax_reference(ref_in, k, renorm)
    assert torch.equal(ids.long().sort(-1).values, ids_ref.long().sort(-1).values)
    if dtype == torch.float32:
        assert torch.equal(ids, ids_ref)  # bf16 logits tie; ties may be ordered differently
    o, o_ref = ids.long().argsort(-1), ids_ref.long().argsort(-1)
    assert torch.allclose(w.gather(1, o), w_ref.gather(1, o_ref), atol=1e-5, rtol=1e-4)
    g = torch.randn_like(w)
    w.backward(g.gather(1, o.argsort(-1)) if False else g)
    # the same upstream gradient per selected expert, whatever the order of ties
    g_ref = torch.zeros_like(g).scatter(1, o_ref, g.gather(1, o))
    w_ref.backward(g_ref)
    assert _rel(logits.grad, ref_in.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)


def test_grouped_sigmoid_topk():
    torch.manual_seed(1)
    logits = torch.randn(257, 256, device="cuda")
    bias = torch.randn(256, device="cuda") * 0.1
    w, ids = moe_ops.grouped_sigmoid_topk(logits, bias, 8, 4, 8, True, 2.5)
    w_ref, ids_ref = moe_ops.grouped_sigmoid_topk_reference(logits, bias, 8, 4, 8, True, 2.5)
    assert torch.equal(ids.long().sort(-1).values, ids_ref.long().sort(-1).values)
    order, order_ref = ids.long().argsort(-1), ids_ref.long().argsort(-1)
    assert torch.allclose(w.gather(1, order), w_ref.gather(1, order_ref), atol=1e-5)


def _plan_equal(a, b):
    return all(torch.equal(getattr(a, n).cpu(), getattr(b, n).cpu())
               for n in ("expert_rows", "tile_expert", "row_route", "route_row", "counts"))


@pytest.mark.parametrize("tokens,E,k,e_lo,e_count", [(1000, 128, 8, 0, 128), (1000, 128, 8, 32, 16), (5, 8, 2, 0, 8),
                                                     (4096, 128, 8, 0, 128), (64, 128, 8, 0, 128), (65, 128, 8, 112, 16)])
def test_align_matches_reference(tokens, E, k, e_lo, e_count):
    torch.manual_seed(2)
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(tokens)]).to(torch.int32).cuda()
    plan = moe_ops.align(ids, e_lo, e_count)
    ref = moe_ops.align(ids.cpu(), e_lo, e_count)
    assert _plan_equal(plan, ref)


@pytest.mark.parametrize("tokens,E,k,H,inter", [(1000, 128, 8, 2048, 768), (77, 8, 2, 256, 128), (3, 16, 4, 512, 64)])
def test_moe_layer_fwd_bwd(tokens, E, k, H, inter):
    torch.manual_seed(3)
    dev = "cuda"
    x = torch.randn(tokens, H, device=dev).to(torch.bfloat16).requires_grad_()
    w1 = (torch.randn(E, 2 * inter, H, device=dev) * 0.03).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(E, H, inter, device=dev) * 0.03).to(torch.bfloat16).requires_grad_()
    logits = torch.randn(tokens, E, device=dev)
    rw, ids = moe_ops.topk_softmax(logits, k, True)
    rw = rw.detach().requires_grad_()

    def run(x_, w1_, w2_, rw_, ref: bool):
        plan = moe_ops.align(ids if not ref else ids.cpu(), 0, E)
        if ref:
            plan = moe_ops.MoePlan(plan.tokens, plan.k, plan.e_count, plan.max_rows, *(t.to(dev) for t in (
                plan.expert_rows, plan.tile_expert, plan.row_route, plan.route_row, plan.counts)))
            xs = moe_ops._gather_rows_reference(x_, plan)
            gu = _ref_grouped(xs, w1_, plan)
            a = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
            ys = _ref_grouped(a, w2_, plan)
            return _ref_combine(ys, plan, rw_)
        from areno_b200.ops import activation

        xs = moe_ops.permute(x_, plan)
        gu = moe_ops.grouped_linear(xs, w1_, plan)
        a = activation.silu_and_mul(gu)
        ys = moe_ops.grouped_linear(a, w2_, plan)
        return moe_ops.combine(ys, plan, rw_)

    out = run(x, w1, w2, rw, False)
    xr, w1r, w2r, rwr = (t.detach().float().requires_grad_() for t in (x, w1, w2, rw))
    out_ref = run(xr, w1r, w2r, rwr, True)
    assert _rel(out, out_ref) < 2e-2
    g = torch.randn_like(out)
    out.backward(g)
    out_ref.backward(g.float())
    _lib.check_status()
    assert _rel(x.grad, xr.grad) < 3e-2
    assert _rel(rw.grad, rwr.grad) < 3e-2
    assert _rel(w1.grad, w1r.grad) < 3e-2
    assert _rel(w2.grad, w2r.grad) < 3e-2


def _ref_grouped(xs, w, plan):
    out = torch.zeros((plan.max_rows, w.shape[1]), dtype=torch.float32, device=xs.device)
    er = plan.expert_rows.tolist()
    for e in range(plan.e_count):
        lo, n = er[2 * e], er[2 * e + 1]
        if n:
            out[lo:lo + n] = xs[lo:lo + n].float() @ w[e].float().t()
    return out


def _ref_combine(ys, plan, weights):
    ro = plan.route_row.long().view(plan.tokens, plan.k)
    valid = (ro >= 0).float()
    rows = ys[ro.clamp(min=0)]
    return (rows * (weights * valid)[:, :, None]).sum(1)


def test_wgrad_accumulates_into_main_grad():
    torch.manual_seed(4)
    E, N, K, T, k = 8, 256, 128, 200, 2
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32).cuda()
    plan = moe_ops.align(ids, 0, E)
    xs = moe_ops.permute(torch.randn(T, K, device="cuda").to(torch.bfloat16), plan)
    w = (torch.randn(E, N, K, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    w.main_grad = torch.ones(E, N, K, device="cuda")
    ys = moe_ops.grouped_linear(xs, w, plan)
    dys = torch.zeros_like(ys)
    er = plan.expert_rows.view(E, 2).tolist()
    for lo, n in er:
        dys[lo:lo + n] = torch.randn(n, N, device="cuda").to(torch.bfloat16)
    dys = dys * (plan.row_route >= 0)[:, None]
    ys.backward(dys)
    assert w.grad is None and w.grad_added_to_main_grad
    ref = torch.ones(E, N, K, device="cuda")
    for e, (lo, n) in enumerate(er):
        ref[e] += dys[lo:lo + n].float().t() @ xs[lo:lo + n].float()
    assert _rel(w.main_grad, ref) < 1e-2


@pytest.mark.parametrize("routes,E,e_lo,e_count,max_rows,drops", [
    (65536, 128, 16, 16, 4096, True), (262144, 128, 0, 16, 16384, True), (5000, 64, 0, 64, 4096, True),
    (9000, 32, 8, 8, 16384, False)])
def test_three_launch_align_matches_the_single_cta_kernel_with_capacity(routes, E, e_lo, e_count, max_rows, drops):
    """Plan built by count / scan / place kernels against the single-CTA kernel, for a row buffer smaller than the
    static bound (routes are dropped) and with -1 entries (padding of an expert-parallel routing table)."""
    from areno_b200.parallel import ep  # noqa: F401  (registers the capped entry point)

    torch.manual_seed(5)
    ids = torch.randint(0, E, (routes,), dtype=torch.int32, device="cuda")
    ids[torch.rand(routes, device="cuda") < 0.1] = -1
    plans = []
    for name in ("areno_moe_align_capped", "areno_moe_align_par"):
        er = torch.empty(2 * e_count, dtype=torch.int32, device="cuda")
        te = torch.empty(max_rows // 128, dtype=torch.int32, device="cuda")
        rr = torch.empty(max_rows, dtype=torch.int32, device="cuda")
        ro = torch.empty(routes, dtype=torch.int32, device="cuda")
        cnt = torch.empty(e_count, dtype=torch.int32, device="cuda")
        dropped = torch.zeros(1, dtype=torch.int32, device="cuda")
        args = [ids.data_ptr(), routes, e_lo, e_count, max_rows, er.data_ptr(), te.data_ptr(), rr.data_ptr(), ro.data_ptr(),
                cnt.data_ptr(), dropped.data_ptr()]
        if name.endswith("par"):
            scratch = moe_ops.align_scratch(routes, e_count, "cuda")
            args.append(scratch.data_ptr())
        _lib.call(name, *args, _lib.stream())
        torch.cuda.synchronize()
        plans.append([t.cpu() for t in (er, te, rr, ro, cnt, dropped)])
    for a, b in zip(*plans):
        assert torch.equal(a, b)
    assert (int(plans[0][5]) > 0) == drops                 # the small buffers really dropped routes, the last case none


def test_inference_fast_paths_match_the_training_path():
    """Without gradients the MoE layer copies and activates only the routed rows and takes its router logits from
    the small fp32 kernel; the layer output must equal the grad-enabled path (which fills the padding rows)."""
    from areno_b200.ops import activation

    torch.manual_seed(9)
    t, E, k, H, inter = 48, 32, 4, 512, 256
    x = torch.randn(t, H, device="cuda").to(torch.bfloat16)
    gate = torch.randn(E, H, device="cuda") * 0.1
    w1 = (torch.randn(E, 2 * inter, H, device="cuda") * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(E, H, inter, device="cuda") * 0.03).to(torch.bfloat16)

    def layer():
        logits = moe_ops.router_logits(x, gate)
        wts, ids = moe_ops.topk_softmax(logits, k, True)
        plan = moe_ops.align(ids, 0, E)
        xs = moe_ops.permute(x, plan)
        a = activation.silu_and_mul(moe_ops.grouped_linear(xs, w1, plan), plan.row_route)
        return logits, moe_ops.combine(moe_ops.grouped_linear(a, w2, plan), plan, wts)

    with torch.enable_grad():
        ref_logits, ref = layer()
    with torch.no_grad():
        logits, out = layer()
    torch.cuda.synchronize()
    assert torch.allclose(logits, ref_logits, atol=2e-4, rtol=1e-4)
    assert torch.allclose(logits, x.float() @ gate.t(), atol=2e-4, rtol=1e-4)
    assert torch.isfinite(out).all() and _rel(out, ref) < 1e-3
