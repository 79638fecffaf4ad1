"""Single-kernel micro-benchmarks of the hot ops at the benchmark model's shapes.

    python -m areno_b200.utils.microbench --case gemm_fwd --iters 5 --warmup 3
    python -m areno_b200.utils.microbench --list

Every case builds inputs larger than the 126 MB L2 (or rotates between several weight copies when
one operand is smaller), times ``iters`` launches with CUDA events after ``warmup`` launches, and
prints achieved TFLOP/s and GB/s together with the fraction of the measured roofline found in
``MEASURED_PEAKS.json`` at the repository root (cuBLAS bf16 burst throughput and STREAM-style copy
bandwidth of this machine).  The same command line is what the profiler captures are taken from;
cases hold at most a few GB on the device.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0}


def load_peaks() -> tuple[dict, str]:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            data = json.load(f)
        return {"bf16_tflops": float(data["bf16_tflops"]), "hbm_gbs": float(data["hbm_gbs"])}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


def _bf16(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


# Each case returns (callable, flops_per_call, bytes_per_call, note)
def case_gemm_fwd():
    from ..ops import gemm

    m, n, k = 4096, 37888, 3584  # gate_up projection of one 4096-token micro-batch
    a, w = _bf16(m, k), _bf16(n, k, scale=0.02)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    return (lambda: gemm.gemm(a, w, out=out)), 2.0 * m * n * k, 2.0 * (m * k + n * k + m * n), f"M={m} N={n} K={k}"


def case_gemm_dgrad():
    from ..ops import gemm

    m, n, k = 4096, 3584, 37888  # dX = dY[M, 37888] @ W[37888, 3584]
    dy, w = _bf16(m, k), _bf16(k, n, scale=0.02)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    return (lambda: gemm.gemm(dy, w, out=out, b_mn=True)), 2.0 * m * n * k, 2.0 * (m * k + n * k + m * n), \
        f"M={m} N={n} K={k} (B MN-major)"


def case_gemm_wgrad():
    from ..ops import gemm

    tokens, n, k = 4096, 37888, 3584  # dW[N, K] += dY^T[N, T] @ X[T, K], fp32 accumulate
    dy, x = _bf16(tokens, n), _bf16(tokens, k)
    out = torch.zeros(n, k, device="cuda", dtype=torch.float32)
    return (lambda: gemm.gemm(dy, x, out=out, a_mn=True, b_mn=True, accumulate=True)), 2.0 * tokens * n * k, \
        2.0 * tokens * (n + k) + 8.0 * n * k, f"M={n} N={k} K={tokens} (A, B MN-major; fp32 accumulate)"


def _rotating_weights(n, k, min_bytes=400e6):
    copies = max(2, int(min_bytes // (n * k * 2)) + 1)
    return [_bf16(n, k, scale=0.02) for _ in range(copies)]


def case_gemm_decode_down():
    from ..ops import gemm

    m, n, k = 64, 3584, 18944
    a = _bf16(m, k)
    ws = _rotating_weights(n, k)
    state = {"i": 0}

    def run():
        w = ws[state["i"] % len(ws)]
        state["i"] += 1
        return gemm.gemm(a, w)

    return run, 2.0 * m * n * k, 2.0 * (n * k + m * k + m * n), f"M={m} N={n} K={k} split-K, {len(ws)} weight copies"


def case_gemm_decode_gate_up():
    from ..ops import gemm

    m, n, k = 64, 37888, 3584
    a = _bf16(m, k)
    ws = _rotating_weights(n, k)
    state = {"i": 0}

    def run():
        w = ws[state["i"] % len(ws)]
        state["i"] += 1
        return gemm.gemm(a, w)

    return run, 2.0 * m * n * k, 2.0 * (n * k + m * k + m * n), f"M={m} N={n} K={k}, {len(ws)} weight copies"


def case_splitk_rmsnorm():
    from ..ops import gemm, norm

    m, n, k = 64, 3584, 3584
    a, res, nw = _bf16(m, k), _bf16(m, n), torch.ones(n, device="cuda", dtype=torch.bfloat16)
    ws = _rotating_weights(n, k)
    state = {"i": 0}

    def run():
        w = ws[state["i"] % len(ws)]
        state["i"] += 1
        part = gemm.gemm_partials(a, w)
        if isinstance(part, gemm.SplitKPartial):
            return norm.splitk_residual_rmsnorm(part, res, nw, 1e-6)
        return norm.rmsnorm(part, nw, 1e-6, residual=res)

    return run, 2.0 * m * n * k, 2.0 * (n * k + m * k + 3 * m * n), f"o_proj M={m} N={n} K={k} + fold/residual/RMSNorm"


def _attn_inputs(lens, hq=28, hkv=4, d=128):
    from ..ops import attention as attn

    t = sum(lens)
    qkv = _bf16(t, (hq + 2 * hkv) * d)
    q = qkv[:, : hq * d].unflatten(1, (hq, d))
    k = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
    v = qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d))
    meta = attn.build_varlen_meta(lens, device="cuda")
    flops = sum(4.0 * hq * d * (n * (n + 1) / 2) for n in lens)  # causal QK^T and PV
    return q, k, v, meta, flops


def case_attn_fwd():
    from ..ops import attention as attn

    lens = [1536] * 16  # 24.6k tokens: q/k/v 180 MB
    q, k, v, meta, flops = _attn_inputs(lens)
    out = torch.empty_like(q.contiguous())
    return (lambda: attn.attention_forward(q, k, v, meta, 128 ** -0.5, True, 0, out=out)), flops, \
        2.0 * sum(lens) * 128 * (28 * 2 + 8), f"{len(lens)} x {lens[0]} tokens, 28 q / 4 kv heads, d=128, causal"


def case_attn_bwd():
    from ..ops import attention as attn

    lens = [1536] * 16
    q, k, v, meta, flops = _attn_inputs(lens)
    o, lse = attn.attention_forward(q, k, v, meta, 128 ** -0.5, True, 0)
    do = torch.randn_like(o)
    dq, dk, dv = torch.empty_like(o), torch.empty_like(k.contiguous()), torch.empty_like(v.contiguous())
    return (lambda: attn.attention_backward(q, k, v, o, do, lse, meta, 128 ** -0.5, True, 0, dq, dk, dv)), 2.5 * flops, \
        2.0 * sum(lens) * 128 * (28 * 4 + 16), "backward of attn_fwd (delta + dK/dV + dQ kernels)"


def case_paged_decode(fp8: bool = False, ctx: int = 1024):
    from ..ops import paged_attention as pa

    b, hq, hkv, d = 64, 28, 4, 128
    pages_per_seq = ctx // pa.PAGE
    num_pages = b * pages_per_seq * 4  # 4x the live pages: 1 GB of bf16 KV so that L2 cannot hold it
    kc, vc, ks, vs = pa.alloc_kv_cache(num_pages, hkv, d, "cuda", fp8=fp8)
    if fp8:
        kc.random_(0, 120)
        vc.random_(0, 120)
    else:
        kc.normal_()
        vc.normal_()
    perm = torch.randperm(num_pages, device="cuda").to(torch.int32)
    tables = [perm[i * b * pages_per_seq:(i + 1) * b * pages_per_seq].view(b, pages_per_seq).contiguous() for i in range(4)]
    lens = torch.full((b,), ctx, dtype=torch.int32, device="cuda")
    q = _bf16(b, hq, d)
    state = {"i": 0}

    def run():
        bt = tables[state["i"] % 4]
        state["i"] += 1
        return pa.paged_decode(q, kc, vc, ks, vs, bt, lens, d ** -0.5, max_context=ctx)

    elt = 1 if fp8 else 2
    return run, 4.0 * b * hq * d * ctx, 2.0 * b * hkv * ctx * d * elt, f"B={b} ctx={ctx} 28 q / 4 kv heads, {'fp8' if fp8 else 'bf16'} pages"


def case_sampler():
    from ..ops import sampling

    b, v = 64, 152064
    logits = torch.randn(b * 8, v, device="cuda")  # 8 row groups, 311 MB
    uid = torch.arange(b, device="cuda", dtype=torch.int64)
    gen = torch.zeros(b, dtype=torch.int32, device="cuda")
    state = {"i": 0}

    def run():
        i = state["i"] % 8
        state["i"] += 1
        return sampling.sample(logits[i * b:(i + 1) * b], 1.0, -1, 1.0, gen_count=gen, seed=1, row_uid=uid)

    return run, 0.0, 4.0 * b * v, f"B={b} V={v} fp32 logits, temperature 1"


def case_adamw():
    from ..ops import optim

    n = 256 * 1024 * 1024  # 1 GiB per fp32 tensor
    master, m, v, g = (torch.zeros(n, device="cuda") for _ in range(4))
    g.normal_()
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    return (lambda: optim.adamw_fp32(master, m, v, g, out, 1e-5, 0.9, 0.999, 1e-8, 0.01, 1)), 0.0, \
        n * (4 * 4 + 3 * 4 + 2.0), f"{n} elements, fp32 master/m/v"


def case_moe_grouped():
    from ..ops import moe

    tokens, e, k, h, inter = 4096, 128, 8, 2048, 768
    ids = torch.stack([torch.randperm(e, device="cuda")[:k] for _ in range(tokens)]).to(torch.int32)
    plan = moe.align(ids, 0, e)
    xs = moe.permute(_bf16(tokens, h), plan)
    w = _bf16(e, 2 * inter, h, scale=0.02)
    return (lambda: moe.grouped_linear(xs, w, plan)), 2.0 * tokens * k * 2 * inter * h, \
        2.0 * (e * 2 * inter * h + tokens * k * (h + 2 * inter)), f"{tokens} tokens x top-{k} of {e} experts, {h}->{2 * inter}"


def case_decode_step(batch: int = 64, ctx: int = 512):
    """One decode step of the benchmark model (Qwen2.5-7B shape, random weights) replayed from its CUDA graph:
    ``batch`` running sequences with ``ctx`` cached tokens each."""
    from ..engine.config import ModelConfig
    from ..engine.inference import InferenceEngine, SamplingParams
    from ..models.dense import DenseCausalLM, init_weights
    from ..ops.paged_attention import PAGE
    from ..parallel.context import single_process_context

    dev = torch.device("cuda", 0)
    single_process_context(dev)
    cfg = ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                      num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, head_dim=128, qkv_bias=True,
                      qk_norm=False, tie_word_embeddings=False, rope_theta=1e6)
    model = DenseCausalLM(cfg, device=dev)
    init_weights(model, 0)
    eng = InferenceEngine(model, cfg.vocab_size, dev, max_slots=batch, max_model_len=ctx + 512)
    eng.begin(SamplingParams(temperature=1.0), (), 16)
    with torch.no_grad():
        eng.active[:batch] = 1
        eng.seq_len[:batch] = ctx
        eng.max_new[:batch] = 4096
        eng.block_table.copy_(torch.arange(batch * eng.max_pages, dtype=torch.int32, device=dev).view(batch, eng.max_pages))
    weights = sum(p.numel() * p.element_size() for n, p in model.named_parameters() if not n.startswith("embed"))
    kv = 28 * 2 * batch * ctx * 4 * 128 * 2
    assert eng.max_pages * PAGE >= ctx + 64

    def run():
        with torch.no_grad():
            eng._decode(batch, eng._context_bucket(ctx + 1))

    return run, 0.0, float(weights + kv), f"B={batch} ctx={ctx}, 7B shape, graph replay (weights {weights / 1e9:.1f} GB + KV {kv / 1e9:.2f} GB)"


def case_train_microbatch(layers: int = 4, lens=(1536, 1408, 1152)):
    """Forward + backward of one packed training micro-batch (4096 tokens in three sequences) through ``layers``
    layers of the benchmark model plus its LM head and the per-token log-prob op, activations kept (no recompute):
    the kernel sequence of a training step at a size that a profiler can walk."""
    from ..engine.config import ModelConfig
    from ..engine.logprobs import lm_head_logprobs
    from ..models.dense import DenseCausalLM, TrainMeta, init_weights
    from ..ops.attention import build_varlen_meta
    from ..parallel.context import single_process_context

    dev = torch.device("cuda", 0)
    single_process_context(dev)
    cfg = ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                      num_hidden_layers=layers, num_attention_heads=28, num_key_value_heads=4, head_dim=128, qkv_bias=True,
                      qk_norm=False, tie_word_embeddings=False, rope_theta=1e6)
    model = DenseCausalLM(cfg, device=dev)
    init_weights(model, 0)
    t = sum(lens)
    ids = torch.randint(3, cfg.vocab_size, (t,), device=dev)
    pos = torch.cat([torch.arange(n, device=dev) for n in lens])
    keep = torch.ones(t, dtype=torch.bool, device=dev)
    ends = torch.tensor(lens, device=dev).cumsum(0) - 1
    keep[ends] = False                                   # the last token of a sequence predicts nothing
    aidx = keep.nonzero().squeeze(1)
    targets = ids.index_select(0, aidx + 1)
    meta = TrainMeta(build_varlen_meta(list(lens), device=dev), activation_checkpointing=True, checkpoint_layers=0)
    weight = torch.randn(aidx.numel(), device=dev)
    for prm in model.parameters():          # as in the trainer: weight gradients accumulate into fp32 buffers
        prm.main_grad = torch.zeros(prm.shape, dtype=torch.float32, device=dev)
        prm.grad_added_to_main_grad = False
    per_layer = 3584 * (4608 + 3584 + 3 * 18944)
    flops = 6.0 * t * per_layer * layers + 8.0 * aidx.numel() * 3584 * 152064   # LM head: logits recomputed in backward

    def run():
        out = model(ids, pos, meta)
        lp = lm_head_logprobs(model.lm_head, out.hidden_states.index_select(0, aidx), targets, 4096)
        (lp * weight).sum().backward()
        for prm in model.parameters():
            prm.grad = None

    return run, flops, 0.0, f"{t} tokens in {len(lens)} sequences, {layers} layers of the 7B shape + LM head, forward + backward"


def case_decode_step_moe(batch: int = 32, ctx: int = 1024, layers: int = 4):
    """One decode step of ``layers`` layers of the Qwen3-30B-A3B shape (128 experts, top 8, all experts on this
    GPU) replayed from its CUDA graph: the kernel sequence of a mixture-of-experts decode step without the
    expert-parallel exchange."""
    from ..engine.config import ModelConfig
    from ..engine.inference import InferenceEngine, SamplingParams
    from ..models.dense import init_weights
    from ..models.moe import MoeCausalLM
    from ..parallel.context import single_process_context

    dev = torch.device("cuda", 0)
    single_process_context(dev)
    cfg = ModelConfig(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                      num_hidden_layers=layers, num_attention_heads=32, num_key_value_heads=4, head_dim=128, qkv_bias=False,
                      qk_norm=True, tie_word_embeddings=False, rope_theta=1e6, num_experts=128, num_experts_per_tok=8,
                      moe_intermediate_size=768, norm_topk_prob=True)
    model = MoeCausalLM(cfg, device=dev)
    init_weights(model, 0)
    eng = InferenceEngine(model, cfg.vocab_size, dev, max_slots=batch, max_model_len=ctx + 512)
    eng.begin(SamplingParams(temperature=1.0), (), 16)
    with torch.no_grad():
        eng.active[:batch] = 1
        eng.seq_len[:batch] = ctx
        eng.max_new[:batch] = 4096
        eng.block_table.copy_(torch.arange(batch * eng.max_pages, dtype=torch.int32, device=dev).view(batch, eng.max_pages))
    weights = sum(p.numel() * p.element_size() for n, p in model.named_parameters() if not n.startswith("embed"))

    def run():
        with torch.no_grad():
            eng._decode(batch, eng._context_bucket(ctx + 1))

    return run, 0.0, float(weights), f"B={batch} ctx={ctx}, {layers} MoE layers (128 experts local) + LM head, graph replay"


def _lightning_inputs(seqs=16, length=1024, h=16, d=128):
    t = seqs * length
    wide = _bf16(t, 3 * h * d, scale=0.5)
    q, k, v = (wide[:, i * h * d:(i + 1) * h * d].unflatten(1, (h, d)) for i in range(3))
    slope = torch.rand(h, device="cuda") * 0.3 + 0.01
    cu = torch.arange(0, t + 1, length, dtype=torch.int32, device="cuda")
    return q, k, v, slope, cu, [length] * seqs


def case_lightning_fwd():
    from ..ops import linear_attn as la

    q, k, v, slope, cu, lens = _lightning_inputs()
    t, h, d = q.shape
    return (lambda: la.lightning_recurrent(q, k, v, slope, cu, d ** -0.5)), 4.0 * t * h * d * d, 4.0 * t * h * d * 2, \
        f"{len(lens)} x {lens[0]} tokens, {h} heads, d={d} (sequential scan per sequence and head)"


def case_lightning_bwd():
    from ..ops import linear_attn as la

    q, k, v, slope, cu, lens = _lightning_inputs()
    t, h, d = q.shape
    qg, kg, vg = (x.detach().contiguous().requires_grad_() for x in (q, k, v))
    o = la.lightning_attention(qg, kg, vg, slope, lens, d ** -0.5, cu=cu)
    g = torch.randn_like(o)

    def run():
        torch.autograd.grad(o, (qg, kg, vg), g, retain_graph=True)

    return run, 12.0 * t * h * d * d, 7.0 * t * h * d * 2, "backward of lightning_fwd (three scans in one launch)"


def case_group_norm_gate():
    from ..ops import linear_attn as la

    rows, g, w = 16384, 4, 512
    x, gate = _bf16(rows, g * w), _bf16(rows, g * w)
    wt = torch.ones(g, w, device="cuda")
    return (lambda: la.group_rmsnorm_sigmoid_gate(x, gate, wt, 1e-6)), 0.0, 3.0 * rows * g * w * 2, \
        f"{rows} rows x {g} groups of {w} (group RMSNorm x sigmoid gate, forward)"


def case_gemm_gated():
    from ..ops import gemm

    m, inter, k = 4096, 18944, 3584
    x, w = _bf16(m, k), _bf16(2 * inter, k, scale=k ** -0.5)

    def run():
        with torch.no_grad():
            gemm.gated_linear(x, w, "silu")

    return run, 2.0 * m * 2 * inter * k, 2.0 * (m * k + 2 * inter * k + m * inter), \
        f"M={m} I={inter} K={k}: gate/up GEMM with SiLU(gate) * up in the epilogue"


def case_lm_head_lse(fused: bool = True):
    """LM-head scoring of one 4096-row chunk: statistics from the GEMM epilogue (no logits tensor) against GEMM to
    bf16 logits followed by the row-statistics kernel."""
    from ..ops import gemm, logprob

    m, n, k = 4096, 152064, 3584
    h, w = _bf16(m, k), _bf16(n, k, scale=0.02)
    t = torch.randint(0, n, (m,), device="cuda")

    def run_fused():
        logprob.fused_head_stats(h, w, t, 0, n)

    def run_unfused():
        logits = gemm.gemm(h, w)
        logprob._stats(logits, t, 0)

    nbytes = 2.0 * (m * k + n * k) + (0.0 if fused else 2.0 * 2.0 * m * n)
    return (run_fused if fused else run_unfused), 2.0 * m * n * k, nbytes, \
        f"M={m} N={n} K={k}: " + ("log-sum-exp statistics in the epilogue" if fused else "bf16 logits written and read back")


def _tp_local_gemm(m, n, k):
    from ..ops import gemm

    a = _bf16(m, k)
    ws = _rotating_weights(n, k)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    state = {"i": 0}

    def run():
        w = ws[state["i"] % len(ws)]
        state["i"] += 1
        gemm.gemm(a, w, out=out)

    return run, 2.0 * m * n * k, 2.0 * (m * k + n * k + m * n), f"M={m} N={n} K={k} (per-rank shape of a TP decode step)"


CASES = {
    "decode_step": case_decode_step,
    "train_microbatch": case_train_microbatch, "decode_step_moe": case_decode_step_moe,
    "lm_head_lse": case_lm_head_lse, "lm_head_unfused": lambda: case_lm_head_lse(False),
    # per-rank GEMM shapes of a tensor-parallel decode step of the 7B model: tp 4 with 256 pooled rows, tp 8 with 512
    "tp4_gate_up": lambda: _tp_local_gemm(256, 9472, 3584), "tp4_down": lambda: _tp_local_gemm(256, 3584, 4736),
    "tp4_qkv": lambda: _tp_local_gemm(256, 1152, 3584), "tp4_o": lambda: _tp_local_gemm(256, 3584, 896),
    "tp8_gate_up": lambda: _tp_local_gemm(512, 4736, 3584), "tp8_down": lambda: _tp_local_gemm(512, 3584, 2368),
    "tp8_qkv": lambda: _tp_local_gemm(512, 768, 3584), "tp8_o": lambda: _tp_local_gemm(512, 3584, 512),
    "lightning_fwd": case_lightning_fwd, "lightning_bwd": case_lightning_bwd, "group_norm_gate": case_group_norm_gate,
    "gemm_gated": case_gemm_gated,
    "gemm_fwd": case_gemm_fwd, "gemm_dgrad": case_gemm_dgrad, "gemm_wgrad": case_gemm_wgrad,
    "gemm_decode_down": case_gemm_decode_down, "gemm_decode_gate_up": case_gemm_decode_gate_up,
    "splitk_rmsnorm": case_splitk_rmsnorm, "attn_fwd": case_attn_fwd, "attn_bwd": case_attn_bwd,
    "paged_decode": case_paged_decode, "paged_decode_fp8": lambda: case_paged_decode(True),
    "paged_decode_4k": lambda: case_paged_decode(False, 4096), "paged_decode_fp8_4k": lambda: case_paged_decode(True, 4096),
    "paged_decode_256": lambda: case_paged_decode(False, 256), "paged_decode_fp8_256": lambda: case_paged_decode(True, 256), "sampler": case_sampler,
    "adamw": case_adamw, "moe_grouped": case_moe_grouped,
}


def run_case(name: str, iters: int, warmup: int, profile_last: bool = False, graph: bool = False) -> dict:
    fn, flops, nbytes, note = CASES[name]()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        # kernels of a few tens of microseconds: an eager loop measures the host's launch rate, so the `iters` calls
        # are captured once and the graph is replayed (as the decode step does)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(iters):
                    fn()
            for _ in range(2):
                g.replay()
            side.synchronize()
            reps = 5
            start.record(side)
            for _ in range(reps):
                g.replay()
            end.record(side)
            side.synchronize()
        us = start.elapsed_time(end) * 1e3 / (iters * reps)
        note += " [graph replay]"
    else:
        start.record()
        for _ in range(iters):
            fn()
        end.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(end) * 1e3 / iters
    if profile_last:
        # one more call inside a profiler range (for `ncu --profile-from-start off`); never timed
        torch.cuda.profiler.start()
        fn()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    peaks, origin = load_peaks()
    out = {"case": name, "shape": note, "us_per_call": round(us, 2), "peaks": origin}
    if flops:
        tf = flops / us / 1e6
        out["tflops"] = round(tf, 1)
        out["frac_of_bf16_peak"] = round(tf / peaks["bf16_tflops"], 3)
    gbs = nbytes / us / 1e3
    out["gb_per_s"] = round(gbs, 1)
    out["frac_of_hbm_peak"] = round(gbs / peaks["hbm_gbs"], 3)
    from ..ops import _lib

    _lib.check_status()
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--case", default="all")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="capture the timed calls into one CUDA graph and time its replay (for kernels shorter than a launch)")
    ap.add_argument("--profile-last", action="store_true",
                    help="run one extra, untimed call per case inside a cudaProfilerStart/Stop range")
    args = ap.parse_args(argv)
    if args.list:
        print("\n".join(CASES))
        return 0
    names = list(CASES) if args.case == "all" else [c.strip() for c in args.case.split(",")]
    for name in names:
        print(json.dumps(run_case(name, args.iters, args.warmup, args.profile_last, args.graph)), flush=True)
        torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
