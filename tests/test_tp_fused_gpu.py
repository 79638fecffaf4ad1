"""Two, four and eight GPUs: the fused row-parallel path (GEMM partial in the symmetric heap, then one
kernel that reduces over the group, adds the residual, normalises and publishes the rows to every rank)
against NCCL + PyTorch fp32, with plain peer loads / stores and, where the fabric offers a multicast
object, with ``multimem`` instructions.  Each size is skipped on a box with fewer GPUs.  Every rank
leaves only after a group barrier, with nothing in flight, and releases its heap first."""

from __future__ import annotations

import os
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

        from areno_b200.ops import _lib
        from areno_b200.parallel.context import init_parallel
        from areno_b200.parallel.symm import setup_tp_comm

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        ctx = init_parallel(rank, world, tp_size=world, master_port=port, device=dev, timeout_s=120)
        H, eps = 3584, 1e-6
        comm = setup_tp_comm(ctx, H, 4096)
        has_mc = bool(comm.heap.mc_base)      # exercise both paths wherever a multicast mapping exists
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        shared = torch.Generator(device=dev).manual_seed(7)
        errs = []
        # (multimem, one-shot): plain two-shot and one-shot always; both multimem variants where a mapping exists
        modes = [(False, "0"), (False, "1")] + ([(True, "0"), (True, "1")] if has_mc else [])
        # decode-shaped (split-K), a single row, fewer rows than ranks, multi-tile, a prefill-sized chunk, and an
        # embedding-style call without residual
        shapes = [(64, 1792), (1, 9472), (3, 512), (300, 1792), (128, 9472), (2500, 896), (64, 1792), (17, 512)]
        for use_mc, oneshot in modes:
            comm.use_mc = use_mc
            os.environ["ARENO_TP_ONESHOT"] = oneshot
            for i, (rows, k_local) in enumerate(shapes):
                x = torch.randn(rows, k_local, device=dev, generator=g).to(torch.bfloat16)
                w = (torch.randn(H, k_local, device=dev, generator=g) * 0.05).to(torch.bfloat16)
                res = torch.randn(rows, H, device=dev, generator=shared).to(torch.bfloat16) if i != 7 else None
                nw = (1 + 0.1 * torch.randn(H, device=dev, generator=shared)).to(torch.bfloat16)
                part = comm.row_linear(x, w)
                y, h = comm.reduce_rmsnorm(part, res, nw, eps)
                y, h = y.clone(), h.clone()
                partial = (x.float() @ w.float().t()).to(torch.bfloat16).float()
                dist.all_reduce(partial, group=ctx.tp_group)
                h_ref = (partial + (res.float() if res is not None else 0.0)).to(torch.bfloat16).float()
                y_ref = h_ref * torch.rsqrt(h_ref.pow(2).mean(-1, keepdim=True) + eps) * nw.float()
                torch.cuda.synchronize()
                errs.append((_rel(h, h_ref), _rel(y, y_ref)))
                # every rank must hold bit-identical results
                both = [torch.empty_like(h) for _ in range(world)]
                dist.all_gather(both, h, group=ctx.tp_group)
                assert all(torch.equal(both[0], b) for b in both[1:])
                both = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(both, y, group=ctx.tp_group)
                assert all(torch.equal(both[0], b) for b in both[1:])
        os.environ.pop("ARENO_TP_ONESHOT", None)
        comm.barrier()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        ret[rank] = {"errs": errs, "multicast": has_mc, "heap": comm.heap.kind}
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()
    finally:
        try:
            if comm is not None:
                comm.close()      # synchronize, group barrier, unbind and unmap: nobody leaves with work in flight
        except BaseException:  # noqa: BLE001
            pass


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_row_parallel_reduce_rmsnorm_matches_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
    for r in range(world):
        assert isinstance(ret[r], dict), ret[r]
        for h_err, y_err in ret[r]["errs"]:
            assert h_err < 8e-3 and y_err < 8e-3, ret[r]
