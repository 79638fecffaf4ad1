"""Further benchmark configurations, selected with ``python bench.py --config NAME`` (the default,
``grpo7b``, lives in ``bench.py``).  Each prints one JSON line in the same format.

``serve8b``  Serving / decode: Llama-3-8B-shaped model (32 layers, hidden 4096, 32 query / 8 KV heads, SwiGLU
             14336, vocab 128256, random init), tensor parallel over all GPUs of the job, fp8 (e4m3) paged KV.
             Concurrent-batch sweep 1 / 16 / 64 / 256, prompt lengths uniform in [512, 4096], 512 output tokens
             per request with EOS ignored.  Per batch size: p50 time to first token, p50 time per output token
             and decode tokens per second (generated tokens after the first, divided by the time from the last
             first-token to the end).  ``value`` is the decode rate at the largest batch that ran.
``dpo7b``    DPO on the Qwen2.5-7B shape, data parallel over all GPUs: 32 preference pairs per GPU (256 at eight
             GPUs), shared prompt of 1024 uniform-random tokens, chosen and rejected responses of 1024 tokens each,
             beta 0.1, a frozen reference role scored before the update, micro-batches of one pair (4096 tokens),
             one AdamW step.  ``value`` is sequence tokens per second through reference scoring + training.

Both use synthetic token ids and random-init weights; timing is CUDA events on the launching stream after warm-up,
max over ranks.
"""

from __future__ import annotations

import json
import os
import sys
import time

import numpy as np

LLAMA8B = dict(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
               num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               rms_norm_eps=1e-5, rope_theta=500_000.0, max_position_embeddings=8192, qkv_bias=False,
               qk_norm=False, tie_word_embeddings=False)


def _env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


def _max_over_ranks(values, device, world):
    import torch
    import torch.distributed as dist

    t = torch.tensor(values, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


# --------------------------------------------------------------------------------------- serving
def run_serve(args) -> None:
    import torch
    import torch.distributed as dist

    import bench
    from areno_b200.engine.config import EngineConfig, ModelConfig, RuntimeConfig
    from areno_b200.engine.inference import SamplingParams
    from areno_b200.engine.worker import RankWorker
    from areno_b200.ops import _lib as klib
    from areno_b200.parallel.context import init_parallel, use_context

    rank, world, local_rank = _env()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    tp = world
    init_parallel(rank, world, tp_size=tp, device=device)
    model_kw = dict(LLAMA8B)
    batches, pmin, pmax, new_tokens = [1, 16, 64, 256], 512, 4096, 512
    if args.small:
        model_kw.update(hidden_size=512, intermediate_size=1536, num_hidden_layers=4, num_attention_heads=8,
                        num_key_value_heads=8, vocab_size=32000)
        batches, pmin, pmax, new_tokens = [1, 8], 32, 128, 32
    kv_dtype = os.environ.get("ARENO_BENCH_KV", "fp8")
    mcfg = ModelConfig(**model_kw)
    max_len = (pmax + new_tokens + 63) // 64 * 64
    cfg = EngineConfig(model=mcfg, tp_size=tp, dp_size=1, devices=list(range(world)), dummy_load=True,
                       runtime=RuntimeConfig(max_model_len=max_len, kv_dtype=kv_dtype, max_prefill_tokens=16384),
                       max_running_seqs=max(batches), decode_progress_interval_s=0.0, seed=1234)
    worker = RankWorker(cfg, device)
    worker.prepare_for_rollout()
    params = SamplingParams(temperature=1.0, top_p=1.0, top_k=-1)
    sampler = bench.ClockSampler(local_rank)
    sweep = []
    launches0 = None
    with use_context(worker.rollout_ctx), torch.no_grad():
        eng = worker.inference_engine(max(batches), max_len)
        for b in batches:
            rng = np.random.default_rng(77 + b)      # every TP rank draws the same prompts
            prompts = [rng.integers(3, mcfg.vocab_size, size=int(n)).tolist() for n in rng.integers(pmin, pmax + 1, size=b)]
            for timed in (False, True):             # one untimed pass per batch size (graphs, allocator), then the timed one
                if timed and launches0 is None:
                    sampler.start()
                    launches0 = klib.launch_count
                eng.begin(params, (), new_tokens)
                rids = [eng.add_request(p) for p in prompts]
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                first: dict[int, float] = {}
                done_at: dict[int, float] = {}
                while not eng.idle:
                    finished = eng.step()
                    pending_first = len(first) < b
                    if pending_first or finished:
                        torch.cuda.synchronize()
                    now = time.perf_counter()
                    if pending_first:
                        for r in rids:
                            req = eng._requests[r]
                            if r not in first and req.slot >= 0 and eng.sched.slot_request(req.slot) == r \
                                    and eng.sched.slot_seq_len(req.slot) >= len(req.context):
                                first[r] = now - t0
                    for req in finished:
                        done_at[req.rid] = now - t0
                for req in eng._poll(block=True, drain=True):
                    done_at[req.rid] = time.perf_counter() - t0
                torch.cuda.synchronize()
                total = time.perf_counter() - t0
                if not timed:
                    continue
                for r in rids:
                    done_at.setdefault(r, total)
                    first.setdefault(r, total)
                ttft = sorted(first[r] for r in rids)
                tpot = sorted((done_at[r] - first[r]) / max(new_tokens - 1, 1) for r in rids)
                t_decode = total - max(ttft)
                gen = sum(len(eng._requests[r].tokens or []) for r in rids)
                vals = _max_over_ranks([ttft[len(ttft) // 2], tpot[len(tpot) // 2], t_decode, total], device, world)
                sweep.append({"batch": b, "ttft_p50_ms": round(vals[0] * 1e3, 2), "tpot_p50_ms": round(vals[1] * 1e3, 3),
                              "decode_tok_s": round((gen - b) / max(vals[2], 1e-9), 1),
                              "total_tok_s": round(gen / max(vals[3], 1e-9), 1), "generated": gen,
                              "prompt_tokens": sum(len(p) for p in prompts)})
    clocks = sampler.stop()
    klib.check_status()
    if rank == 0:
        print(json.dumps({
            "metric": "decode tok/s (serving, largest batch of the sweep)", "value": sweep[-1]["decode_tok_s"],
            "unit": "tokens/s", "n_gpus": world, "steps": 1, "warmup": 1, "ms_per_step": None, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "impl": "ours", "sweep": sweep, "clocks": clocks,
            "data": "synthetic (uniform random token ids, random-init weights)",
            "gpu_launches": klib.launch_count - (launches0 or 0),
            "config": {"model": "Llama-3-8B-shaped" if not args.small else "small-debug", "kv_cache": f"{kv_dtype} paged, page 64",
                       "parallelism": f"tp{tp}", "prompt_len": [pmin, pmax], "new_tokens": new_tokens, "batches": batches,
                       "timing": "wall clock with a device synchronize at every first-token and completion event",
                       "l2": "inputs larger than L2 (weights and KV pages streamed every step)"}}), flush=True)
    worker.close()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


# --------------------------------------------------------------------------------------- DPO
def run_dpo(args) -> None:
    import torch
    import torch.distributed as dist
    from functools import partial

    import bench
    from areno_b200.api import Trainer, TrainSequence
    from areno_b200.api.loss_fns import dpo_loss_fn
    from areno_b200.api.roles import ModelRole
    from areno_b200.engine.config import EngineConfig, ModelConfig, OptimizerConfig, RuntimeConfig
    from areno_b200.engine.worker import RankWorker
    from areno_b200.ops import _lib as klib
    from areno_b200.parallel.context import init_parallel

    rank, world, local_rank = _env()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    init_parallel(rank, world, tp_size=1, device=device)
    model_kw = dict(bench.MODEL)
    pairs_per_gpu, prompt_len, resp_len = 32, 1024, 1024
    if args.small:
        model_kw.update(hidden_size=512, intermediate_size=1536, num_hidden_layers=4, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=32000)
        pairs_per_gpu, prompt_len, resp_len = 4, 64, 64
    mcfg = ModelConfig(**model_kw)
    cfg = EngineConfig(model=mcfg, tp_size=1, dp_size=world, devices=list(range(world)), dummy_load=True,
                       optimizer=OptimizerConfig(lr=1e-6, weight_decay=0.01, grad_clip_norm=1.0),
                       runtime=RuntimeConfig(activation_checkpointing=True, max_model_len=prompt_len + resp_len),
                       max_running_seqs=8, decode_progress_interval_s=0.0, seed=1234)
    worker = RankWorker(cfg, device)
    trainer = Trainer.from_worker(worker, world_size=world, eos_ids=(0,))     # pad id for scoring batches
    trainer.ensure_roles({"ref": ModelRole("ref", "", trainable=False)})
    loss_fn = partial(dpo_loss_fn, beta=0.1)
    n_pairs = pairs_per_gpu * world

    def make_batch(step: int):
        rng = np.random.default_rng(4242 + step)
        batch = []
        for _ in range(n_pairs):
            prompt = rng.integers(3, mcfg.vocab_size, size=prompt_len).tolist()
            for _side in range(2):
                resp = rng.integers(3, mcfg.vocab_size, size=resp_len).tolist()
                n = prompt_len + resp_len
                batch.append(TrainSequence(prompt_mask=[True] * prompt_len + [False] * resp_len, tokens=prompt + resp,
                                           logprobs=[0.0] * n, advantages=[0.0] * n, eos_token_id=0))
        return batch

    def one_step(step: int):
        batch = make_batch(step)
        rows = trainer.score_logprobs("ref", [s.tokens for s in batch])
        for seq, ref in zip(batch, rows):
            seq.ref_logprobs = [float(v) for v in ref]
        stats = trainer.train(batch, loss_fn, mini_bs=2 * world)
        return sum(len(s.tokens) for s in batch), stats

    for w in range(args.warmup):
        one_step(w)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = bench.ClockSampler(local_rank)
    sampler.start()
    klib.launch_count = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    tokens, stats = 0, {}
    for s in range(args.steps):
        n, stats = one_step(args.warmup + s)
        tokens += n
    end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ms = _max_over_ranks([start.elapsed_time(end)], device, world)[0]
    klib.check_status()
    if rank == 0:
        print(json.dumps({
            "metric": "DPO step tokens/sec (reference scoring + train)", "value": tokens / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "ours",
            "data": "synthetic (uniform random token ids, random-init weights, frozen reference = copy of the actor)",
            "clocks": clocks, "gpu_launches": klib.launch_count, "last_loss": stats.get("loss"),
            "dpo_accuracy": stats.get("dpo_accuracy"),
            "config": {"model": "Qwen2.5-7B-shaped" if not args.small else "small-debug", "global_batch": 2 * n_pairs,
                       "pairs": n_pairs, "seq_len": prompt_len + resp_len, "beta": 0.1, "micro_batch_tokens": 2 * (prompt_len + resp_len),
                       "parallelism": f"dp{world}, sharded grads + optimizer, frozen reference role resident on the GPU",
                       "l2": "inputs larger than L2 (15 GB of weights streamed every micro-batch)"}}), flush=True)
    worker.close()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)
