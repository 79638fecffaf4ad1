"""Two GPUs: the row-parallel GEMM that pushes its partial into every rank's inbox, and the fused
all-reduce + residual + RMSNorm consumer, against NCCL + PyTorch fp32.  Skipped with fewer than two
GPUs.  NVLS is switched off and the kernels use plain peer stores / local loads."""

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
    try:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        import torch.distributed as dist

        from areno_b200.ops import _lib
        from areno_b200.parallel.context import init_parallel
        from areno_b200.parallel.symm import setup_tp_comm

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        ctx = init_parallel(rank, world, tp_size=world, master_port=port, device=dev, timeout_s=120)
        H, eps = 3584, 1e-6
        comm = setup_tp_comm(ctx, H, 512)
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        shared = torch.Generator(device=dev).manual_seed(7)
        errs = []
        # decode-shaped (split-K fold delivers), a single row, and a multi-tile problem (epilogue delivers)
        for i, (rows, k_local) in enumerate([(64, 1792), (1, 9472), (300, 1792), (128, 9472), (64, 1792), (17, 512)]):
            x = torch.randn(rows, k_local, device=dev, generator=g).to(torch.bfloat16)
            w = (torch.randn(H, k_local, device=dev, generator=g) * 0.05).to(torch.bfloat16)
            res = torch.randn(rows, H, device=dev, generator=shared).to(torch.bfloat16)
            nw = (1 + 0.1 * torch.randn(H, device=dev, generator=shared)).to(torch.bfloat16)
            part = comm.push_linear(x, w)
            y, h = comm.reduce_rmsnorm(part, res, nw, eps)
            partial = (x.float() @ w.float().t()).to(torch.bfloat16).float()
            dist.all_reduce(partial, group=ctx.tp_group)
            h_ref = (partial + res.float()).to(torch.bfloat16).float()
            y_ref = h_ref * torch.rsqrt(h_ref.pow(2).mean(-1, keepdim=True) + eps) * nw.float()
            torch.cuda.synchronize()
            errs.append((_rel(h, h_ref), _rel(y, y_ref)))
            # every rank must hold bit-identical results
            both = [torch.empty_like(h) for _ in range(world)]
            dist.all_gather(both, h, group=ctx.tp_group)
            assert all(torch.equal(both[0], b) for b in both[1:])
        _lib.check_status(dev)
        # a wait that nothing satisfies runs out and reports instead of hanging (rank 0 alone calls)
        ret[rank] = errs
        dist.barrier()
        comm.close()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_push_gemm_and_fused_reduce_rmsnorm_match_nccl():
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], list), ret[r]
        for h_err, y_err in ret[r]:
            assert h_err < 8e-3 and y_err < 8e-3, ret[r]
