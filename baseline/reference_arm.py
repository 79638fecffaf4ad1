"""Reference arm of ``bench.py``: the unmodified reference installed under ``baseline/_ref`` driven
through its own public engine API (``areno.ArenoEngine.from_pretrained`` / ``generate_rollout`` /
``step``) on the same workload as our arm: 64 x N sequences per step, prompt lengths uniform in
[128, 512], 1024 new tokens at temperature 1, seeded-hash reward, GRPO update in micro-batches of
about 4096 tokens per rank, one AdamW step.

Reference limits that shape the run (recorded in the JSON line): the Qwen2.5-7B shape has to be
presented as ``model_type: qwen3`` with ``attention_bias`` on and ``qk_layernorm`` off; 28 Q / 4 KV
heads allow tp in {1, 2, 4} only, and the default layout is tp=1 x dp=N (``ARENO_REF_TP`` picks another); weights are replicated and only the
optimizer state is sharded; there is no separate weight sync because rollout and training share
one module.  The reference runs its workers in its own spawned processes, so the step is timed by
wall clock around its blocking API calls (which return after every rank has finished).
"""

from __future__ import annotations

import json
import os
import sys
import time
import traceback

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _emit(obj):
    print(json.dumps(obj), flush=True)


def _write_random_checkpoint(path: str, model: dict, seed: int = 1234) -> None:
    """Seeded random HF-safetensors checkpoint of the benchmark shape (bf16, normal(0, 0.02))."""
    import torch
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    if os.path.exists(os.path.join(path, "model.safetensors.index.json")):
        return
    h, inter, layers = model["hidden_size"], model["intermediate_size"], model["num_hidden_layers"]
    hq, hkv, d, vocab = (model["num_attention_heads"], model["num_key_value_heads"], model["head_dim"],
                         model["vocab_size"])
    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": vocab, "hidden_size": h,
        "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": hq,
        "num_key_value_heads": hkv, "head_dim": d, "rms_norm_eps": model["rms_norm_eps"],
        "rope_theta": model["rope_theta"], "max_position_embeddings": model["max_position_embeddings"],
        "tie_word_embeddings": False, "attention_bias": True, "qk_layernorm": False, "torch_dtype": "bfloat16",
        "hidden_act": "silu", "sequence_parallel": False,
    }
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=dev).manual_seed(seed)

    def rnd(*shape):
        return (torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()

    weight_map = {}
    shard_id = 0

    def flush(tensors):
        nonlocal shard_id
        shard_id += 1
        name = f"model-{shard_id:05d}.safetensors"
        save_file(tensors, os.path.join(path, name))
        for k in tensors:
            weight_map[k] = name

    flush({"model.embed_tokens.weight": rnd(vocab, h)})
    for i in range(layers):
        p = f"model.layers.{i}"
        flush({
            f"{p}.input_layernorm.weight": torch.ones(h, dtype=torch.bfloat16),
            f"{p}.post_attention_layernorm.weight": torch.ones(h, dtype=torch.bfloat16),
            f"{p}.self_attn.q_proj.weight": rnd(hq * d, h), f"{p}.self_attn.q_proj.bias": torch.zeros(hq * d, dtype=torch.bfloat16),
            f"{p}.self_attn.k_proj.weight": rnd(hkv * d, h), f"{p}.self_attn.k_proj.bias": torch.zeros(hkv * d, dtype=torch.bfloat16),
            f"{p}.self_attn.v_proj.weight": rnd(hkv * d, h), f"{p}.self_attn.v_proj.bias": torch.zeros(hkv * d, dtype=torch.bfloat16),
            f"{p}.self_attn.o_proj.weight": rnd(h, hq * d),
            f"{p}.mlp.gate_proj.weight": rnd(inter, h), f"{p}.mlp.up_proj.weight": rnd(inter, h),
            f"{p}.mlp.down_proj.weight": rnd(h, inter),
        })
    flush({"model.norm.weight": torch.ones(h, dtype=torch.bfloat16), "lm_head.weight": rnd(vocab, h)})
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)


def _build_packs(torch, rows, responses, logprobs, advantages, rows_per_pack: int, pad_id: int = 0):
    packs = []
    for start in range(0, len(rows), rows_per_pack):
        idx = list(range(start, min(start + rows_per_pack, len(rows))))
        width = max(len(rows[i]) + len(responses[i]) for i in idx)
        ids = torch.full((len(idx), width), pad_id, dtype=torch.long)
        pmask = torch.ones((len(idx), width), dtype=torch.bool)
        lp = torch.zeros((len(idx), width), dtype=torch.float32)
        adv = torch.zeros((len(idx), width), dtype=torch.float32)
        lens = torch.zeros(len(idx), dtype=torch.int32)
        for r, i in enumerate(idx):
            p, resp = rows[i], responses[i]
            n = len(p) + len(resp)
            ids[r, :n] = torch.tensor(p + resp)
            pmask[r, len(p):n] = False
            lp[r, len(p):n] = torch.tensor(logprobs[i][: len(resp)])
            adv[r, len(p):n] = float(advantages[i])
            lens[r] = n
        packs.append({"input_ids": ids, "labels": ids.clone(), "lengths": lens, "prompt_mask": pmask, "logprobs": lp,
                      "advantages": adv})
    return packs


_LAUNCHER_VARS = ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "GROUP_RANK", "LOCAL_WORLD_SIZE",
                  "ROLE_RANK", "ROLE_WORLD_SIZE", "ROLE_NAME", "GROUP_WORLD_SIZE", "OMP_NUM_THREADS")


def _mark(stage: str) -> None:
    """Progress marker on stderr (and in a file the parent reads if the run has to be abandoned)."""
    line = f"[reference-arm {time.strftime('%H:%M:%S')}] {stage}"
    print(line, file=sys.stderr, flush=True)
    path = os.environ.get("ARENO_REF_STAGE_FILE")
    if path:
        with open(path, "w") as f:
            f.write(stage)


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if rank != 0:
        return  # the reference spawns and drives its own per-GPU workers from one driver process
    from baseline.install_reference import ensure_installed

    ok, why = ensure_installed()      # no-op when the build step already installed it
    if not ok:
        _emit({"impl": "reference", "unavailable": f"baseline/_ref is not installed and could not be installed here: {why}"})
        return
    if os.environ.get("ARENO_REF_CHILD") != "1" and (world > 1 or "TORCHELASTIC_RUN_ID" in os.environ):
        _run_isolated(args, max(world, args.gpus))
        return
    # the reference's workers are separate processes: drop the launcher's rendezvous variables
    for k in _LAUNCHER_VARS:
        os.environ.pop(k, None)
    sys.path.insert(0, REF)
    try:
        _run(args, max(world, args.gpus))
    except BaseException as exc:  # report, never crash the driver's round-end run
        tb = traceback.format_exc().strip().splitlines()
        _emit({"impl": "reference", "unavailable": f"reference run failed: {type(exc).__name__}: {str(exc)[:300]}",
               "trace_tail": tb[-6:]})


def _run_isolated(args, n_gpus: int) -> None:
    """Under a multi-rank launcher the reference is driven from a fresh interpreter with none of the
    launcher's environment (its own engine spawns and rendezvouses its workers), and with a deadline:
    a run that does not finish is reported as unavailable with the stage it had reached."""
    import subprocess
    import tempfile

    env = {k: v for k, v in os.environ.items() if k not in _LAUNCHER_VARS and not k.startswith("TORCHELASTIC")}
    env["ARENO_REF_CHILD"] = "1"
    stage_file = tempfile.NamedTemporaryFile(prefix="areno_ref_stage_", delete=False).name
    env["ARENO_REF_STAGE_FILE"] = stage_file
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", str(n_gpus), "--steps",
           str(args.steps), "--warmup", str(args.warmup)] + (["--small"] if args.small else [])
    deadline = float(os.environ.get("ARENO_REF_DEADLINE_S", 480 + 60 * (args.steps + args.warmup)))
    try:
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=deadline, start_new_session=True)
    except subprocess.TimeoutExpired as exc:
        stage = open(stage_file).read() if os.path.exists(stage_file) else "start"
        sys.stderr.write((exc.stderr or b"").decode(errors="replace")[-2000:] if isinstance(exc.stderr, bytes) else str(exc.stderr or "")[-2000:])
        _emit({"impl": "reference", "unavailable": f"reference run did not finish within {deadline:.0f} s at {n_gpus} GPUs "
                                                   f"(last stage: {stage})"})
        return
    sys.stderr.write(proc.stderr[-4000:])
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    if lines:
        print(lines[-1], flush=True)
    else:
        _emit({"impl": "reference", "unavailable": f"reference child exited with code {proc.returncode} and no result line"})


def _run(args, n_gpus: int) -> None:
    import torch

    import bench  # workload constants and synthetic-data helpers shared by both arms

    import areno  # noqa: F401  (the reference package under baseline/_ref)
    from areno import ArenoEngine, OptimizerConfig, RuntimeConfig, SamplingParams
    from areno.api.loss_fns.grpo import grpo_loss_fn

    model = dict(bench.MODEL)
    new_tokens, pmin, pmax, n_prompts = bench.NEW_TOKENS, bench.PROMPT_MIN, bench.PROMPT_MAX, bench.PROMPTS_PER_GPU
    if args.small:
        model.update(hidden_size=512, intermediate_size=1536, num_hidden_layers=4, num_attention_heads=4,
                     num_key_value_heads=2, vocab_size=32000)
        new_tokens, pmin, pmax = 64, 32, 96
    ckpt = os.path.join("/tmp", f"areno_ref_ckpt_{'small' if args.small else '7b'}")
    t0 = time.time()
    _mark("writing checkpoint")
    _write_random_checkpoint(ckpt, model)
    ckpt_s = time.time() - t0
    _mark(f"starting engine on {n_gpus} GPU(s)")
    attn_backend = os.environ.get("ARENO_REF_ATTN", "flash")
    # Layout of the reference: tp must divide the 4 KV heads and the GPU count.  tp=1 x dp=N is the default
    # (ARENO_REF_TP selects tp 2 or 4 for comparison runs).
    ref_tp = int(os.environ.get("ARENO_REF_TP", "1"))
    if ref_tp not in (1, 2, 4) or n_gpus % ref_tp != 0:
        ref_tp = 1
    ref_dp = n_gpus // ref_tp
    engine = ArenoEngine.from_pretrained(
        ckpt, tp_size=ref_tp, dp_size=ref_dp, devices=list(range(n_gpus)),
        optimizer_config=OptimizerConfig(lr=1e-6, betas=(0.9, 0.999), weight_decay=0.01, grad_clip_norm=1.0),
        runtime_config=RuntimeConfig(attn_backend=attn_backend, activation_checkpointing=True),
        loss_fn=grpo_loss_fn)
    _mark("engine ready")
    params = SamplingParams(temperature=1.0, top_p=1.0, top_k=0, suppress_special_tokens=False)
    rows_per_rank = n_prompts * bench.GROUP

    def one_step(step: int):
        rows = []
        for r in range(n_gpus):
            prompts = bench.make_prompts(step, r, model["vocab_size"], n_prompts, pmin, pmax)
            rows.extend(p for p in prompts for _ in range(bench.GROUP))
        _mark(f"step {step}: rollout")
        engine.begin_rollout_session()
        out = engine.generate_rollout(rows, max_new_tokens=new_tokens, max_running_prompts=rows_per_rank * n_gpus,
                                      eos_token_id=None, sampling_params=params)
        engine.end_rollout_session()
        responses = out.response_ids
        resp_lp = []
        lp_t = out.logprobs
        for i, resp in enumerate(responses):
            # padded [rows, max_response] tensor: the first len(resp) entries of a row are its log-probs
            resp_lp.append(lp_t[i, : len(resp)].tolist())
        rewards = np.array([bench.hash_reward(t) for t in responses])
        adv = bench.group_advantages(rewards, bench.GROUP)
        # ~3 sequences (about 4096 tokens) per rank per micro-batch, rows strided over DP by the engine
        packs = _build_packs(torch, rows, responses, resp_lp, adv, rows_per_pack=3 * ref_dp)
        _mark(f"step {step}: train")
        stats = engine.step(packs, gradient_accumulation_steps=None)
        tokens = sum(len(p) + len(t) for p, t in zip(rows, responses))
        last = stats[-1]
        loss = float(getattr(last, "loss", 0.0) if not isinstance(last, dict) else last.get("loss", 0.0))
        return tokens, loss

    try:
        for w in range(args.warmup):
            one_step(w)
        sampler = bench.ClockSampler(0)
        sampler.start()
        t0 = time.time()
        total = 0
        loss = 0.0
        for s in range(args.steps):
            n, loss = one_step(args.warmup + s)
            total += n
        wall = time.time() - t0
        clocks = sampler.stop()
    finally:
        try:
            engine.close()
        except Exception:
            pass
    value = total / wall
    _emit({
        "metric": "RL step rollout+train tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
        "data": "synthetic (uniform random token ids, seeded random-init safetensors checkpoint, seeded-hash reward)",
        "clocks": clocks, "last_loss": loss,
        "e2e": {"value": value, "unit": "tokens/s", "timing": "wall clock around the reference's blocking engine API"},
        "config": {
            "model": "Qwen2.5-7B-shaped (as model_type qwen3, attention_bias on, qk_layernorm off)" if not args.small else "small-debug",
            "global_batch": rows_per_rank * n_gpus, "prompt_len": [pmin, pmax], "new_tokens": new_tokens,
            "seq_len": pmax + new_tokens, "micro_batch_tokens": bench.MICRO_TOKENS,
            "parallelism": f"tp{ref_tp} x dp{ref_dp}, replicated bf16 weights + ZeRO-1 optimizer, attn_backend={attn_backend}",
            "timing": "wall clock around blocking engine calls (workers are separate processes)",
            "checkpoint_write_s": ckpt_s,
        },
    })
