"""Headline benchmark: one GRPO RL step (rollout + train + weight sync) on a Qwen2.5-7B-shaped model.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Per GPU the step does 8 prompts x 8 samples (prompt lengths uniform in [128, 512], uniform random
token ids, 1024 new tokens at temperature 1.0 with EOS ignored), a seeded-hash {0,1} reward,
group-normalised advantages, and a GRPO update over micro-batches of at most 4096 tokens with fp32
gradient accumulation and one AdamW step.  With N > 1 (one process per GPU, launched by
``torch.distributed.run``) the per-GPU work is fixed (weak scaling): 64 x N sequences per step.

Metric: whole-job tokens per second, counting every sequence token (prompt + response) once per
step, i.e. the tokens that went through rollout and were then trained on.

Two numbers are reported: ``value`` is timed with CUDA events around the engine-level step;
``e2e`` is timed by wall clock around the same step driven through the public SDK
(``areno_b200.api.Trainer``), including the pinned host->device copy of the step's token ids and
the device->host read of the rollout results and the loss.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
             num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
             rms_norm_eps=1e-6, rope_theta=1_000_000.0, max_position_embeddings=32768, qkv_bias=True,
             qk_norm=False, tie_word_embeddings=False)
PROMPTS_PER_GPU = 8
GROUP = 8
PROMPT_MIN, PROMPT_MAX = 128, 512
NEW_TOKENS = 1024
MICRO_TOKENS = 4096
BASELINE_PUBLISHED = None  # the reference publishes no number for this metric

# --config moe30b: Qwen3-30B-A3B shape, expert parallel over all ranks, 4 prompts x group 8 per GPU (32 x 8 on 8 GPUs),
# 2048 new tokens.  The full 48 layers need the 8-GPU layout (3.6 G expert parameters per rank with their fp32
# optimizer state); with fewer GPUs the layer count shrinks in proportion so that the per-rank footprint stays.
MOE_MODEL = dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                 num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                 rms_norm_eps=1e-6, rope_theta=1_000_000.0, max_position_embeddings=32768, qkv_bias=False,
                 qk_norm=True, tie_word_embeddings=False, num_experts=128, num_experts_per_tok=8,
                 moe_intermediate_size=768, norm_topk_prob=True)
MOE_PROMPTS_PER_GPU, MOE_NEW_TOKENS = 4, 2048


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="grpo7b", choices=["grpo7b", "moe30b", "serve8b", "dpo7b"],
                    help="grpo7b: the headline RL step (default); moe30b: the same step on a Qwen3-30B-A3B-shaped "
                         "mixture-of-experts model with expert parallelism; serve8b / dpo7b: see bench_extra.py")
    ap.add_argument("--small", action="store_true", help="tiny model / short rollout (functional check only)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--adam-8bit", action="store_true")
    ap.add_argument("--rollout-tp", type=int, default=0,
                    help="TP width of the rollout engine (0: pick automatically; 1: one replica per GPU)")
    return ap.parse_args()


# Rollout TP width per GPU count, from the measured rollout time of each layout on this workload
# (``profiles/bench_7b_grpo_scaling.md``); ``ARENO_BENCH_ROLLOUT_TP`` or ``--rollout-tp`` override it.
ROLLOUT_TP_BY_WORLD = {1: 1, 2: 1, 4: 1, 8: 1}


def pick_rollout_tp(world: int) -> int:
    """Rollout layout for the benchmark model.  28 query / 4 KV heads split evenly over tp 2 and 4; tp 8 uses the
    uneven head split of the rollout-only layout (4 + 3 query heads per KV pair)."""
    env = os.environ.get("ARENO_BENCH_ROLLOUT_TP")
    tp = int(env) if env else ROLLOUT_TP_BY_WORLD.get(world, 1)
    return tp if tp >= 1 and world % tp == 0 else 1


# ------------------------------------------------------------------------- synthetic data
def make_prompts(step: int, rank: int, vocab: int, n_prompts: int, pmin: int, pmax: int) -> list[list[int]]:
    rng = np.random.default_rng(1000003 * step + rank)
    lens = rng.integers(pmin, pmax + 1, size=n_prompts)
    return [rng.integers(3, vocab, size=int(n)).tolist() for n in lens]


def hash_reward(tokens: list[int]) -> float:
    h = 1469598103934665603
    for t in tokens:
        h = ((h ^ (t & 0xFFFFFFFF)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return float((h >> 17) & 1)


def group_advantages(rewards: np.ndarray, group: int) -> np.ndarray:
    r = rewards.reshape(-1, group)
    adv = (r - r.mean(1, keepdims=True)) / (r.std(1, keepdims=True) + 1e-8)
    return adv.reshape(-1)


def build_micro_batches(prompts, responses, logprobs, advantages, micro_tokens: int, groups=None):
    """Padded (B, T) packs holding at most ``micro_tokens`` real tokens: greedy fill in input order, or the given
    ``groups`` of sequence indices."""
    import torch

    if groups is None:
        groups, cur, cur_tokens = [], [], 0
        for i in range(len(prompts)):
            n = len(prompts[i]) + len(responses[i])
            if cur and cur_tokens + n > micro_tokens:
                groups.append(cur)
                cur, cur_tokens = [], 0
            cur.append(i)
            cur_tokens += n
        if cur:
            groups.append(cur)
    packs = []
    for g in groups:
        width = max(len(prompts[i]) + len(responses[i]) for i in g)
        ids = torch.zeros((len(g), width), dtype=torch.int64)
        pmask = torch.ones((len(g), width), dtype=torch.bool)
        lp = torch.zeros((len(g), width), dtype=torch.float32)
        adv = torch.zeros((len(g), width), dtype=torch.float32)
        lens = torch.zeros(len(g), dtype=torch.int64)
        for r, i in enumerate(g):
            p, resp = prompts[i], responses[i]
            n = len(p) + len(resp)
            ids[r, :n] = torch.tensor(p + resp)
            pmask[r, len(p):n] = False
            lp[r, len(p):n] = torch.tensor(logprobs[i])
            adv[r, len(p):n] = float(advantages[i])
            lens[r] = n
        packs.append(dict(input_ids=ids, lengths=lens, prompt_mask=pmask, logprobs=lp, advantages=adv))
    return packs


# ------------------------------------------------------------------------- clocks sampling
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    from areno_b200.api import loss_fns
    from areno_b200.engine.config import EngineConfig, ModelConfig, OptimizerConfig, RuntimeConfig
    from areno_b200.engine.inference import SamplingParams
    from areno_b200.engine.training import balanced_partition, pack_into_bins
    from areno_b200.engine.worker import RankWorker
    from areno_b200.ops import _lib as klib
    from areno_b200.parallel.context import init_parallel

    balance = os.environ.get("ARENO_BENCH_BALANCE", "1") != "0"
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    moe = args.config == "moe30b"
    ep = moe and world > 1
    rollout_tp = 1 if moe else (args.rollout_tp or pick_rollout_tp(world))
    ctx = init_parallel(rank, world, tp_size=1, device=device, rollout_tp_size=rollout_tp, expert_parallel=ep)
    balance = balance or ep      # expert parallel: every rank must run the same number of micro-batches

    model_kw = dict(MOE_MODEL if moe else MODEL)
    new_tokens, pmin, pmax, n_prompts = NEW_TOKENS, PROMPT_MIN, PROMPT_MAX, PROMPTS_PER_GPU
    if moe:
        new_tokens, n_prompts = MOE_NEW_TOKENS, MOE_PROMPTS_PER_GPU
        if world < 8:
            model_kw["num_hidden_layers"] = 6 * world
    if args.small and moe:
        model_kw.update(hidden_size=512, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                        vocab_size=32000, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256)
        new_tokens, pmin, pmax = 64, 32, 96
    elif args.small:
        model_kw.update(hidden_size=512, intermediate_size=1536, num_hidden_layers=4, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=32000)
        new_tokens, pmin, pmax = 64, 32, 96
    mcfg = ModelConfig(**model_kw)
    cfg = EngineConfig(
        model=mcfg, tp_size=1, dp_size=world, rollout_tp_size=None if moe else rollout_tp, expert_parallel=ep,
        devices=list(range(world)), dummy_load=True,
        optimizer=OptimizerConfig(lr=1e-6, betas=(0.9, 0.999), weight_decay=0.01, grad_clip_norm=1.0,
                                  adam_8bit=args.adam_8bit),
        runtime=RuntimeConfig(activation_checkpointing=True, max_model_len=(pmax + new_tokens + 63) // 64 * 64),
        max_running_seqs=n_prompts * GROUP, decode_progress_interval_s=0.0, seed=1234)
    worker = RankWorker(cfg, device)
    worker.loss_fn = loss_fns.grpo_loss_fn
    params = SamplingParams(temperature=1.0, top_p=1.0, top_k=-1)

    phase = {"rollout_s": 0.0, "train_s": 0.0, "host_s": 0.0}

    def one_step(step: int):
        t0 = time.time()
        prompts = make_prompts(step, rank, mcfg.vocab_size, n_prompts, pmin, pmax)
        rows = [p for p in prompts for _ in range(GROUP)]
        t1 = time.time()
        out = worker.rollout(rows, params, eos_token_ids=(), max_new_tokens=new_tokens, progress_interval_s=0.0,
                             gather_tp=True)
        t2 = time.time()
        rewards = np.array([hash_reward(t) for t in out.tokens])
        adv = group_advantages(rewards, GROUP)
        tokens = sum(len(p) + len(t) for p, t in zip(rows, out.tokens))
        seqs = (rows, out.tokens, out.logprobs, [float(a) for a in adv])
        groups = None
        if world > 1 and balance:
            # Deal the job's sequences out again so that every rank trains on the same number of sequences, nearly the
            # same number of tokens, and the same number of micro-batches (the slowest rank sets the step time).
            gathered = [None] * world
            dist.all_gather_object(gathered, seqs)
            flat = [[x for part in gathered for x in part[k]] for k in range(4)]
            lengths = [len(p) + len(t) for p, t in zip(flat[0], flat[1])]
            plan = balanced_partition(lengths, world)
            n_bins = max(len(pack_into_bins([lengths[i] for i in plan[r]], MICRO_TOKENS)) for r in range(world))
            seqs = tuple([col[i] for i in plan[rank]] for col in flat)
            groups = pack_into_bins([lengths[i] for i in plan[rank]], MICRO_TOKENS, n_bins)
        packs = build_micro_batches(seqs[0], seqs[1], seqs[2], seqs[3], MICRO_TOKENS, groups)
        t3 = time.time()
        stats = worker.train(packs)
        torch.cuda.synchronize()
        t4 = time.time()
        if os.environ.get("ARENO_BENCH_VERBOSE"):
            print(f"[bench] rank {rank} step {step}: rollout {t2 - t1:.3f}s train {t4 - t3:.3f}s", file=sys.stderr, flush=True)
        phase["rollout_s"] += t2 - t1
        phase["train_s"] += t4 - t3
        phase["host_s"] += (t1 - t0) + (t3 - t2)
        return tokens, stats[-1]["loss"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Multi-GPU correctness evidence, taken before the first step: one gradient bucket reduced with the peer-memory
    # kernel against NCCL's reduce-scatter, and (tensor-parallel rollout) one fused row-parallel call against
    # GEMM + NCCL all-reduce + RMSNorm.
    checks = {}
    if world > 1:
        err = worker.training_manager().optimizer.self_check_reduce_scatter()
        if err is not None:
            t = torch.tensor([err], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            checks["grad_rs_max_abs"] = float(t[0])
            assert checks["grad_rs_max_abs"] < 1e-3, f"peer-memory gradient reduce-scatter differs from NCCL: {checks}"
        if worker.tp_comm is not None:
            checks["tp_fused_rel"] = worker.tp_comm.self_check()
            checks["tp_heap"] = worker.tp_comm.heap.kind
            checks["tp_multimem"] = bool(worker.tp_comm.use_mc)
            assert checks["tp_fused_rel"] < 1e-2, f"fused row-parallel reduce differs from NCCL: {checks}"
        klib.check_status()
    for w in range(args.warmup):
        one_step(w)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    klib.launch_count = 0
    for k in phase:
        phase[k] = 0.0
    from areno_b200.utils import tracing

    tracing.phase_report()      # ARENO_PHASE_TIMERS=1: drop what the warm-up steps recorded
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.time()
    start.record()
    total_tokens = 0
    loss = 0.0
    for s in range(args.steps):
        n, loss = one_step(args.warmup + s)
        total_tokens += n
    end.record()
    barrier()
    wall = time.time() - t_wall
    clocks = sampler.stop()
    ms = start.elapsed_time(end)
    launches = klib.launch_count
    t = torch.tensor([ms, float(total_tokens), wall], dtype=torch.float64, device=device)
    if world > 1:
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, wall, total_tokens = float(mx[0]), float(mx[2]), float(sm[1])
    value = total_tokens / (ms / 1e3)
    klib.check_status()
    # device-side time of every named phase (CUDA events, max over ranks); only with ARENO_PHASE_TIMERS=1
    phases = tracing.phase_report_max() if tracing.enabled() else None

    e2e = None
    if ep:
        checks["ep_impl"] = ctx.ep_runtime.impl
        checks["ep_dropped_routes"] = ctx.ep_runtime.dropped()
    if not args.no_e2e and not moe:
        e2e = run_e2e(args, worker, mcfg, params, rank, world, device, n_prompts, pmin, pmax, new_tokens)

    if rank == 0:
        result = {
            "metric": "RL step rollout+train tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (value / BASELINE_PUBLISHED) if BASELINE_PUBLISHED else None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights, seeded-hash reward)",
            "impl": "ours", "clocks": clocks, "gpu_launches": launches, "e2e": e2e, "last_loss": loss, "checks": checks,
            "phase_s_per_step": {k: v / args.steps for k, v in phase.items()},
            **({"device_phase_ms_per_step": {k: round(v["ms"] / args.steps, 3) for k, v in sorted(phases.items())}}
               if phases else {}),
            "config": {
                "model": ("small-debug" if args.small else
                          (f"Qwen3-30B-A3B-shaped, {mcfg.num_hidden_layers} of 48 layers" if moe else "Qwen2.5-7B-shaped")),
                "global_batch": n_prompts * GROUP * world,
                "prompts_per_gpu": n_prompts, "group": GROUP, "prompt_len": [pmin, pmax], "new_tokens": new_tokens,
                "seq_len": pmax + new_tokens, "micro_batch_tokens": MICRO_TOKENS,
                "parallelism": (f"ep{world}: 128 experts dealt out over the ranks, tokens exchanged over peer memory in "
                                f"every MoE layer of rollout and training; dense parts dp{world}; " if ep else "")
                               + f"rollout dp{world // rollout_tp} x tp{rollout_tp} (paged bf16 KV, CUDA-graph decode), "
                               f"train dp{world} sharded grads+optimizer, weight sync: "
                               + ("in place (shared buffers)" if rollout_tp == 1 else
                                  "local reshard of the DP replica into the TP shards; row-parallel all-reduce fused with "
                                  "residual + RMSNorm over the symmetric heap"),
                "tokens_counted": "prompt+response tokens per sequence, once per step",
                "train_sharding": ("sequences re-dealt over ranks by token count before training" if world > 1 and balance
                                   else "each rank trains on the sequences it generated"),
                "l2": "inputs larger than L2 (15 GB of weights streamed every decode step / micro-batch)",
                "wall_s_timed_region": wall,
            },
        }
        print(json.dumps(result), flush=True)
    worker.close()
    if world > 1:
        # Leave without tearing the communicators down: captured decode graphs still reference them, and
        # destroying a communicator in that state can block forever.  The barrier keeps ranks together
        # until rank 0 has printed.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_e2e(args, worker, mcfg, params, rank, world, device, n_prompts, pmin, pmax, new_tokens):
    """The same step through the public SDK (``Trainer.rollout_session`` / ``rollout_token_batch`` /
    ``train``) on top of the already-built worker, timed by wall clock.  Every step the SDK path
    copies that step's token ids (prompts for prefill, packed sequences and per-token signals for
    training) from pinned host memory to the device and reads the sampled tokens, their
    log-probs and the loss / metrics back to the host; those bytes are counted from the tensors."""
    import torch
    import torch.distributed as dist
    from functools import partial

    try:
        from areno_b200.api import SamplingParams as ApiParams, Trainer, TrainSequence, grpo_loss_fn
        from areno_b200.api.rewards import compute_group_advantages
    except Exception as exc:  # SDK layer not importable: report honestly
        return {"value": None, "unit": "tokens/s", "error": f"SDK unavailable: {exc}"}
    # SPMD launch: every rank drives the SDK with its own share of the job (its prompts, its sequences); the ranks
    # meet in the collectives of the engine, not in host-side object exchanges
    local = world > 1
    trainer = Trainer.from_worker(worker, world_size=world, local_data=local)
    api_params = ApiParams(temperature=1.0, top_p=1.0, top_k=-1, max_new_tokens=new_tokens, ignore_eos=True)
    loss_fn = partial(grpo_loss_fn, clip_eps=0.2)
    steps = max(1, min(args.steps, 2))
    counters = {"h2d": 0, "d2h": 0}
    wall = {"rollout_call_s": 0.0, "build_batch_s": 0.0, "train_call_s": 0.0}

    def step(i):
        prompts = []
        for r in ([rank] if local else range(world)):
            prompts.extend(make_prompts(10_000 + i, r, mcfg.vocab_size, n_prompts, pmin, pmax))
        t_a = time.time()
        with trainer.rollout_session(sampling_params=api_params):
            results = trainer.rollout_token_batch(prompts, GROUP, api_params)
        t_b = time.time()
        batch = []
        ntok = 0
        for p, res in zip(prompts, results):
            rewards = [hash_reward(s.resp_tokens) for s in res.sequences]
            for s, adv, rew in zip(res.sequences, compute_group_advantages(rewards), rewards):
                n_r = len(s.resp_tokens)
                batch.append(TrainSequence(prompt_mask=[True] * len(p) + [False] * n_r, tokens=p + s.resp_tokens,
                                           logprobs=[0.0] * len(p) + s.resp_logprobs,
                                           advantages=[0.0] * len(p) + [adv] * n_r, reward=rew, eos_token_id=0))
                ntok += len(p) + n_r
        t_c = time.time()
        stats = trainer.train(batch, loss_fn, mini_bs=3 if local else 3 * world)
        t_d = time.time()
        wall["rollout_call_s"] += t_b - t_a
        wall["build_batch_s"] += t_c - t_b
        wall["train_call_s"] += t_d - t_c
        my_share = 1.0 if local else 1.0 / world
        # per rank: prompt ids (int64) for prefill; ids, positions (int64), 2 float32 signals, mask, seq ids for training
        counters["h2d"] += int(my_share * (sum(len(p) for p in prompts) * GROUP * 8 + ntok * (8 + 8 + 4 + 4 + 1 + 8)))
        counters["d2h"] += int(my_share * sum(len(s.resp_tokens) for r in results for s in r.sequences) * (4 + 4)) + 4 * 16
        return ntok, stats

    for w in range(min(max(args.warmup, 1), 2)):      # untimed: the SDK path packs micro-batches of its own shapes
        step(-1 - w)
    counters["h2d"] = counters["d2h"] = 0
    for k in wall:
        wall[k] = 0.0
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.time()
    tokens = 0
    stats = {}
    per_step = []
    for i in range(steps):
        t_s = time.time()
        n, stats = step(i)
        per_step.append(round(time.time() - t_s, 3))
        tokens += n
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    dt = time.time() - t0
    if world > 1:
        t = torch.tensor([dt], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t[0])
        if local:       # every rank counted its own tokens
            n_all = torch.tensor([float(tokens)], dtype=torch.float64, device=device)
            dist.all_reduce(n_all, op=dist.ReduceOp.SUM)
            tokens = float(n_all[0])
    return {"value": tokens / dt, "unit": "tokens/s", "steps": steps, "ms_per_step": dt / steps * 1e3,
            "h2d_bytes_per_step": counters["h2d"] // steps, "d2h_bytes_per_step": counters["d2h"] // steps,
            "timing": "wall clock around Trainer.rollout_token_batch + Trainer.train, max over ranks"
                      + ("; SPMD with rank-local batches (ArenoConfig.spmd_local_data): every rank drives the SDK "
                         "with its own prompts and sequences" if local else ""),
            "step_rollout_time_s": stats.get("step_rollout_time_s"), "step_train_time_s": stats.get("step_train_time_s"),
            "wall_s_per_step_rank0": {k: round(v / steps, 3) for k, v in wall.items()}, "step_wall_s_rank0": per_step,
            "loss": stats.get("loss")}


def main():
    args = parse_args()
    if args.impl == "reference":
        if args.config != "grpo7b":
            print(json.dumps({"impl": "reference", "unavailable": f"the reference arm covers the grpo7b configuration only, not {args.config}"}))
            return
        from baseline.reference_arm import run_reference

        run_reference(args)
        return
    if args.config == "serve8b":
        import bench_extra

        bench_extra.run_serve(args)
    elif args.config == "dpo7b":
        import bench_extra

        bench_extra.run_dpo(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
