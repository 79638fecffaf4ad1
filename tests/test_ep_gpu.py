"""Two, four and eight GPUs: the expert-parallel MoE path (routing tables and tokens exchanged over peer memory, grouped
tcgen05 GEMMs on the expert owners, outputs scattered back) against a single-device fp32 computation on the gathered
tokens with all experts, forward and backward.  Skipped on a box with fewer GPUs."""

from __future__ import annotations

import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def _rank_main(rank, world, port, ret):
    comm = None
    try:
        import torch.distributed as dist

        from areno_b200.ops import _lib, activation, moe as moe_ops
        from areno_b200.parallel.context import init_parallel
        from areno_b200.parallel.ep import EpComm

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        ctx = init_parallel(rank, world, tp_size=1, master_port=port, device=dev, timeout_s=120)
        H, inter, E, k, cap = 512, 256, 8 * world, 4, 256
        e_local = E // world
        comm = EpComm(ctx.dp_group, world, rank, H, cap, k, E, dev, capacity=float(world))   # never drops in this test
        shared = torch.Generator(device=dev).manual_seed(11)
        w_gu_all = (torch.randn(E, 2 * inter, H, device=dev, generator=shared) * 0.05).to(torch.bfloat16)
        w_dn_all = (torch.randn(E, H, inter, device=dev, generator=shared) * 0.05).to(torch.bfloat16)
        w_gu = w_gu_all[rank * e_local:(rank + 1) * e_local].clone().requires_grad_()
        w_dn = w_dn_all[rank * e_local:(rank + 1) * e_local].clone().requires_grad_()
        errs = []
        for step, t in enumerate((cap - 3 * rank, 17 + rank, 130)):      # different token counts on different ranks
            g = torch.Generator(device=dev).manual_seed(100 * step + rank)
            x = torch.randn(t, H, device=dev, generator=g).to(torch.bfloat16).requires_grad_()
            logits = torch.randn(t, E, device=dev, generator=g)
            wts, ids = moe_ops.topk_softmax(logits, k, True)
            wts = wts.detach().requires_grad_()
            dout = torch.randn(t, H, device=dev, generator=g).to(torch.bfloat16)

            rows, plan = comm.dispatch(x, ids)
            gu = moe_ops.grouped_linear(rows, w_gu, plan.moe)
            a = activation.silu_and_mul(gu)
            ys = moe_ops.grouped_linear(a, w_dn, plan.moe)
            out = comm.combine(ys, wts, plan)
            w_gu.grad = w_dn.grad = None
            out.backward(dout)
            torch.cuda.synchronize()

            # reference: every rank recomputes its own tokens with all experts in fp32
            xr = x.detach().float().requires_grad_()
            wr = wts.detach().clone().requires_grad_()
            gu_r = w_gu_all.float().clone().requires_grad_()
            dn_r = w_dn_all.float().clone().requires_grad_()
            acc = torch.zeros(t, H, device=dev)
            for j in range(k):
                e = ids[:, j].long()
                h1 = torch.einsum("th,tnh->tn", xr, gu_r[e]).to(torch.bfloat16).float()
                act = (torch.nn.functional.silu(h1[:, :inter]) * h1[:, inter:]).to(torch.bfloat16).float()
                acc = acc + wr[:, j:j + 1] * torch.einsum("tn,thn->th", act, dn_r[e]).to(torch.bfloat16).float()
            acc.backward(dout.float())
            # expert-weight gradients: the owner accumulates the contributions of every rank's tokens
            gu_grad, dn_grad = gu_r.grad.clone(), dn_r.grad.clone()
            dist.all_reduce(gu_grad, group=ctx.dp_group)
            dist.all_reduce(dn_grad, group=ctx.dp_group)
            sl = slice(rank * e_local, (rank + 1) * e_local)
            errs.append(dict(out=_rel(out, acc), dx=_rel(x.grad, xr.grad), dw=_rel(wts.grad, wr.grad),
                             dgu=_rel(w_gu.grad, gu_grad[sl]), ddn=_rel(w_dn.grad, dn_grad[sl])))
        dropped = comm.dropped()
        comm.barrier()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        ret[rank] = {"errs": errs, "dropped": dropped, "heap": comm.heap.kind, "max_rows": comm.max_rows}
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()
    finally:
        try:
            if comm is not None:
                comm.close()
        except BaseException:  # noqa: BLE001
            pass


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_moe_matches_all_experts_on_one_device(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
    for r in range(world):
        assert isinstance(ret[r], dict), ret[r]
        assert ret[r]["dropped"] == 0
        for e in ret[r]["errs"]:
            assert e["out"] < 2e-2 and e["dx"] < 3e-2 and e["dw"] < 3e-2 and e["dgu"] < 3e-2 and e["ddn"] < 3e-2, ret[r]
