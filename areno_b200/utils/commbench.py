"""Collective micro-benchmarks (launch with ``python -m torch.distributed.run``).

``tp_fused``: the fused row-parallel path of a tensor-parallel decoder block (GEMM partial into the symmetric heap,
then one kernel: reduce over the group + residual add + RMSNorm + publish; ``parallel/symm.py``) against the same
GEMM followed by NCCL ``all_reduce`` and the residual RMSNorm kernel, over all ranks of the job as one TP group, at
decode and prefill row counts.  The roofline of a call is the slower of the GEMM FLOPs at the measured cuBLAS
bf16 rate and the bytes that have to enter each GPU over NVLink at the measured peer-copy rate: ``rows x H`` bf16 for
the one-shot reduce with multimem, ``tp - 1`` times that with plain loads, ``3 (tp - 1) / tp`` for the two-shot scheme
(reduce-scatter of the partial plus all-gather of the residual stream and the normalised rows).

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


def _timed(fn, iters: int, warmup: int, group, graph: bool = False) -> float:
    """Milliseconds per call of ``fn`` (CUDA events on the launching stream, max over ranks).  With ``graph`` the call
    is captured four times into one CUDA graph and the graph is replayed, so that microsecond-scale kernels are
    timed as they run inside a captured decode step and not at the rate the host can launch them."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    per = 1
    run = fn
    if graph:
        per = 4
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(per):
                fn()
        run = g.replay
        run()
        torch.cuda.synchronize()
        dist.barrier(group=group)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        run()
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end) / (iters * per)], device="cuda")
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


def bench_tp_fused(ctx, rows: int, hidden: int, k_full: int, iters: int, warmup: int, comm, peaks: dict) -> dict:
    from ..ops import gemm, norm as norm_ops

    tp, dev = ctx.tp_size, ctx.device
    k_local = k_full // tp
    g = torch.Generator(device=dev).manual_seed(11 + ctx.tp_rank)
    x = torch.randn(rows, k_local, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(hidden, k_local, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    res = torch.randn(rows, hidden, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).to(torch.bfloat16)
    nw = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)   # larger than L2: weights come from HBM every call

    def fused():
        flush.zero_()
        part = comm.row_linear(x, w)
        comm.reduce_rmsnorm(part, res, nw, 1e-6)

    def fused_collective_only():
        part = comm.new_partial(rows)
        comm.reduce_rmsnorm(part, res, nw, 1e-6)

    def nccl():
        flush.zero_()
        y = gemm.gemm(x, w)
        dist.all_reduce(y, group=ctx.tp_group)
        norm_ops.rmsnorm(y, nw, 1e-6, residual=res)

    buf = torch.empty(rows, hidden, device=dev, dtype=torch.bfloat16)

    def nccl_collective_only():
        dist.all_reduce(buf, group=ctx.tp_group)
        norm_ops.rmsnorm(buf, nw, 1e-6, residual=res)

    def flush_only():
        flush.zero_()

    g = rows <= 1024      # decode-sized calls live inside captured graphs; time them that way
    t_flush = _timed(flush_only, iters, warmup, ctx.tp_group, g)
    out = {"case": "tp_fused", "tp": tp, "rows": rows, "hidden": hidden, "k_local": k_local,
           "multimem": bool(comm.multimem(rows)), "one_shot": bool(comm.one_shot(rows)), "heap": comm.heap.kind,
           "timed_in_cuda_graph": g}
    t_f = _timed(fused, iters, warmup, ctx.tp_group, g) - t_flush
    t_n = _timed(nccl, iters, warmup, ctx.tp_group, g) - t_flush
    t_fc = _timed(fused_collective_only, iters, warmup, ctx.tp_group, g)
    t_nc = _timed(nccl_collective_only, iters, warmup, ctx.tp_group, g)
    flops = 2.0 * rows * hidden * k_local
    if comm.one_shot(rows):      # every rank takes in the finished sums (multimem) or tp - 1 remote partials
        link_bytes = (1.0 if comm.multimem(rows) else float(tp - 1)) * rows * hidden * 2
    else:
        link_bytes = 3.0 * (tp - 1) / tp * rows * hidden * 2
    weight_bytes = 2.0 * hidden * k_local
    t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), link_bytes / (PEER_COPY_GBS * 1e9),
                 weight_bytes / (peaks["hbm_gbs"] * 1e9)) * 1e3
    t_roof_coll = link_bytes / (PEER_COPY_GBS * 1e9) * 1e3
    out.update({"fused_us": round(t_f * 1e3, 1), "nccl_us": round(t_n * 1e3, 1), "speedup": round(t_n / t_f, 2),
                "roofline_us": round(t_roof * 1e3, 1), "fused_frac_of_roofline": round(t_roof / t_f, 3),
                "reduce_kernel_us": round(t_fc * 1e3, 1), "nccl_allreduce_norm_us": round(t_nc * 1e3, 1),
                "collective_roofline_us": round(t_roof_coll * 1e3, 1),
                "collective_frac_of_link": round(t_roof_coll / t_fc, 3)})
    return out


def bench_tp_layer(ctx, rows: int, iters: int, warmup: int, comm, ctx_len: int = 768) -> dict:
    """Device time of every kernel group of one tensor-parallel decoder block of the benchmark model at decode
    shapes (``rows`` pooled sequences, ``ctx_len`` cached tokens each), each group captured four times into a CUDA
    graph and replayed: where a decode step of the TP rollout spends its time."""
    from ..engine.config import ModelConfig
    from ..models.dense import DecoderLayer, InferMeta
    from ..ops import activation, gemm, paged_attention as pa
    from ..parallel.symm import TpPartial

    dev = ctx.device
    mcfg = ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                       num_hidden_layers=1, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                       rms_norm_eps=1e-6, rope_theta=1e6, qkv_bias=True, qk_norm=False)
    layer = DecoderLayer(mcfg, 0, torch.bfloat16, dev)
    for p in layer.parameters():
        p.requires_grad_(False)
        if p.dim() >= 2:
            p.normal_(0.0, 0.02)
        else:
            p.fill_(1.0 if p.numel() == mcfg.hidden_size else 0.0)
    attn = layer.attn
    pages = (ctx_len + pa.PAGE) // pa.PAGE + 1
    attn.kv_cache = pa.alloc_kv_cache(rows * pages, attn.hkv, attn.d, dev, False)
    table = torch.arange(rows * pages, dtype=torch.int32, device=dev).view(rows, pages)
    lens = torch.full((rows,), ctx_len + 1, dtype=torch.int32, device=dev)
    pos = torch.full((rows,), ctx_len, dtype=torch.int32, device=dev)
    slots = (table[:, ctx_len // pa.PAGE] * pa.PAGE + ctx_len % pa.PAGE).to(torch.int32)
    meta = InferMeta(mode="decode", slot_mapping=slots, block_table=table, seq_lens=lens, max_context=ctx_len + 64)
    h = (torch.randn(rows, mcfg.hidden_size, device=dev) * 0.5).to(torch.bfloat16)
    res = h.clone()
    out: dict = {"case": "tp_layer", "tp": ctx.tp_size, "rows": rows, "ctx": ctx_len, "multimem": bool(comm.multimem(rows)),
                 "one_shot": bool(comm.one_shot(rows))}
    state: dict = {}

    def qkv_attend():
        state["a"] = attn.attend(h, pos, meta)

    def o_proj():
        state["po"] = attn.o(state["a"])

    def reduce_norm(key):
        def run():
            part = state[key]
            if isinstance(part, TpPartial):
                part = TpPartial(comm, comm.next_slot(), part.rows, part.local)   # a fresh slot per replayed call
                state["y"], state["r"] = comm.reduce_rmsnorm(part, res, layer.post_norm.weight, 1e-6)
        return run

    def gate_up_act():
        gu = layer.mlp.gate_up(h)
        state["act"] = activation.silu_and_mul(gu)

    def down():
        state["pd"] = layer.mlp.down(state["act"])

    with torch.no_grad():
        for name, fn in (("qkv_rope_attention", qkv_attend), ("o_proj", o_proj), ("reduce_norm_after_o", reduce_norm("po")),
                         ("gate_up_act", gate_up_act), ("down_proj", down), ("reduce_norm_after_down", reduce_norm("pd"))):
            out[name + "_us"] = round(_timed(fn, iters, warmup, ctx.tp_group, graph=True) * 1e3, 1)
    out["layer_us"] = round(sum(v for k, v in out.items() if k.endswith("_us")), 1)
    return out


def _peaks() -> dict:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--case", default="grad_rs", choices=["grad_rs", "tp_fused", "tp_layer"])
    ap.add_argument("--rows", type=int, nargs="*", default=[64, 256, 512, 2048, 4096])
    ap.add_argument("--hidden", type=int, default=3584)
    ap.add_argument("--k", type=int, nargs="*", default=[18944, 3584], help="full (unsharded) input widths")
    ap.add_argument("--multimem", type=int, default=-1, help="1 / 0 forces the multimem or the plain peer path")
    ap.add_argument("--oneshot", type=int, default=-1, help="1 / 0 forces the one-shot or the two-shot reduce")
    ap.add_argument("--mib", type=int, nargs="*", default=[256, 1024])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    from ..parallel.context import init_parallel

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    ctx = init_parallel(rank, world, tp_size=world if args.case in ("tp_fused", "tp_layer") else 1,
                        master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"),
                        master_port=int(os.environ.get("MASTER_PORT", "29500")), device=torch.device("cuda", local))
    if args.case == "tp_layer":
        from ..ops import _lib
        from ..parallel.symm import setup_tp_comm

        comm = setup_tp_comm(ctx, args.hidden, max(max(args.rows), 512))
        for rows in args.rows:
            out = bench_tp_layer(ctx, rows, args.iters, args.warmup, comm)
            if rank == 0:
                print(json.dumps(out), flush=True)
        _lib.check_status()
        comm.close()
        dist.barrier()
        os._exit(0)
    if args.case == "tp_fused":
        from ..ops import _lib
        from ..parallel.symm import setup_tp_comm

        comm = setup_tp_comm(ctx, args.hidden, max(args.rows))
        has_mc = bool(comm.heap.mc_base)
        modes = ([True, False] if has_mc else [False]) if args.multimem < 0 else [bool(args.multimem) and has_mc]
        peaks = _peaks()
        if args.oneshot >= 0:
            os.environ["ARENO_TP_ONESHOT"] = str(args.oneshot)
        for use_mc in modes:
            comm.use_mc = use_mc
            for k_full in args.k:
                for rows in args.rows:
                    out = bench_tp_fused(ctx, rows, args.hidden, k_full, args.iters, args.warmup, comm, peaks)
                    out["peaks"] = peaks["source"]
                    if rank == 0:
                        print(json.dumps(out), flush=True)
        _lib.check_status()
        comm.close()
        dist.barrier()
        os._exit(0)
    for mib in args.mib:
        out = bench_grad_rs(ctx, mib, args.iters, args.warmup)
        if rank == 0:
            print(json.dumps(out), flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    raise SystemExit(main())
