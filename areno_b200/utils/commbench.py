"""Collective micro-benchmarks over the data-parallel group (launch with ``python -m torch.distributed.run``).

``grad_rs``: reduce-scatter of fp32 gradient buckets over peer memory (``parallel/grad_comm.py``) against
NCCL's ``reduce_scatter_tensor`` on the same sizes.  Timed with CUDA events on the launching stream after
warm-up, max over ranks; bandwidth is the bytes each rank must pull over NVLink, ``(n - 1) / n`` of the
bucket, divided by that time, and the fraction is of the measured peer-copy rate of this machine
(770 GB/s per direction).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

PEER_COPY_GBS = 770.0


def _timed(fn, iters: int, warmup: int, group) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end) / iters], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
    return float(ms)


def bench_grad_rs(ctx, mib: int, iters: int, warmup: int) -> dict:
    from ..ops import _lib
    from ..parallel.grad_comm import GradComm

    n, rank, dev = ctx.dp_size, ctx.dp_rank, ctx.device
    elems = mib * (1 << 20) // 4 // (4 * n) * (4 * n)
    comm = GradComm(ctx.dp_group, n, rank, elems, dev)
    comm.grads.normal_()

    def fused():
        comm.begin_step()
        comm.launch(0, 0, elems // n)
        comm.finish()

    flat = torch.randn(elems, device=dev)

    def nccl():
        lo = rank * (elems // n)
        dist.reduce_scatter_tensor(flat[lo:lo + elems // n], flat, group=ctx.dp_group)

    t_fused = _timed(fused, iters, warmup, ctx.dp_group)
    t_nccl = _timed(nccl, iters, warmup, ctx.dp_group)
    _lib.check_status()
    comm.close()
    pulled = 4.0 * elems * (n - 1) / n
    return {"case": "grad_rs", "ranks": n, "bucket_mib": round(4.0 * elems / (1 << 20), 1),
            "fused_ms": round(t_fused, 3), "nccl_ms": round(t_nccl, 3),
            "fused_gbs_per_rank": round(pulled / t_fused / 1e6, 1), "nccl_gbs_per_rank": round(pulled / t_nccl / 1e6, 1),
            "fused_frac_of_peer_copy": round(pulled / t_fused / 1e6 / PEER_COPY_GBS, 3)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--mib", type=int, nargs="*", default=[256, 1024])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    from ..parallel.context import init_parallel

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    ctx = init_parallel(rank, world, tp_size=1, master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"),
                        master_port=int(os.environ.get("MASTER_PORT", "29500")), device=torch.device("cuda", local))
    for mib in args.mib:
        out = bench_grad_rs(ctx, mib, args.iters, args.warmup)
        if rank == 0:
            print(json.dumps(out), flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    raise SystemExit(main())
