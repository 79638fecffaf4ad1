"""Decayed linear attention (forward scan, backward scans), the gated group norm, and the Bailing model on a
B200 against their PyTorch references."""

from __future__ import annotations

import pytest
import torch

from areno_b200.ops import _lib, linear_attn as la

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.detach().float() - b.detach().float()).norm() / b.detach().float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("h,d", [(4, 128), (3, 64), (2, 32)])
def test_lightning_forward_backward(h, d):
    torch.manual_seed(0)
    lens = [37, 5, 120, 1]
    t = sum(lens)
    wide = (0.5 * torch.randn(t, 3 * h * d + 16, device="cuda")).to(torch.bfloat16)     # q, k, v as strided views
    q, k, v = (wide[:, i * h * d:(i + 1) * h * d].unflatten(1, (h, d)) for i in range(3))
    slope = torch.rand(h, device="cuda") * 0.3 + 0.01
    cu = torch.tensor([0, 37, 42, 162, 163], dtype=torch.int32, device="cuda")
    scale = d ** -0.5
    # inference scan with per-slot state: sequences 1 and 3 continue from cached state
    slots = torch.tensor([2, 0, 5, 1], dtype=torch.int32, device="cuda")
    fresh = torch.tensor([1, 0, 1, 0], dtype=torch.int32, device="cuda")
    cache = torch.randn(6, h, d, d, device="cuda") * 0.1
    init = [None, cache[0].clone(), None, cache[1].clone()]
    ref, finals = la.lightning_attention_reference(q, k, v, slope, lens, scale, init)
    out = la.lightning_recurrent(q, k, v, slope, cu, scale, state_cache=cache, slots=slots, fresh=fresh)
    _lib.check_status()
    assert _rel(out, ref) < 1e-2
    for i, s in enumerate([2, 0, 5, 1]):
        assert _rel(cache[s], finals[i]) < 1e-3
    # training: forward from zero state and the three backward scans
    qg, kg, vg = (x.detach().clone().requires_grad_() for x in (q, k, v))
    o = la.lightning_attention(qg, kg, vg, slope, lens, scale, cu=cu)
    qr, kr, vr = (x.detach().float().requires_grad_() for x in (q, k, v))
    orf, _ = la.lightning_attention_reference(qr, kr, vr, slope, lens, scale)
    assert _rel(o, orf) < 1e-2
    g = torch.randn_like(o)
    o.backward(g)
    orf.backward(g.float())
    assert _rel(qg.grad, qr.grad) < 1.5e-2 and _rel(kg.grad, kr.grad) < 1.5e-2 and _rel(vg.grad, vr.grad) < 1.5e-2


@pytest.mark.parametrize("rows,g,w", [(100, 4, 512), (7, 16, 128), (513, 3, 40)])
def test_group_rmsnorm_sigmoid_gate(rows, g, w):
    torch.manual_seed(1)
    x = torch.randn(rows, g * w, device="cuda").to(torch.bfloat16).requires_grad_()
    wide = torch.randn(rows, g * w + 32, device="cuda").to(torch.bfloat16)
    gate = wide[:, : g * w].detach().requires_grad_()
    wt = (1 + 0.1 * torch.randn(g, w, device="cuda")).requires_grad_()
    y = la.group_rmsnorm_sigmoid_gate(x, gate, wt, 1e-6)
    xr, gr, wr = (a.detach().float().requires_grad_() for a in (x, gate, wt))
    yr = la.group_rmsnorm_sigmoid_gate_reference(xr, gr, wr, 1e-6)
    assert _rel(y, yr) < 8e-3
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(gate.grad, gr.grad) < 1e-2 and _rel(wt.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("mla", [False, True])
def test_bailing_engine_matches_full_forward_and_trains(mla):
    from areno_b200.api import loss_fns
    from areno_b200.engine.config import EngineConfig, ModelConfig, OptimizerConfig, RuntimeConfig
    from areno_b200.engine.inference import SamplingParams
    from areno_b200.engine.worker import RankWorker
    from areno_b200.models.dense import TrainMeta
    from areno_b200.ops.attention import build_varlen_meta
    from areno_b200.parallel.context import single_process_context

    dev = torch.device("cuda", 0)
    single_process_context(dev)
    kw = dict(kv_lora_rank=64, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128) if mla else \
        dict(qk_nope_head_dim=32, qk_rope_head_dim=32, v_head_dim=64)
    cfg = ModelConfig(
        model_type="bailing_moe_linear_v2", vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=5,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, qk_norm=True, qkv_bias=False, layer_group_size=2,
        partial_rotary_factor=0.5, num_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1, routed_scaling_factor=2.5,
        first_k_dense_replace=1, moe_intermediate_size=128, num_shared_experts=1, group_norm_size=4,
        moe_router_bias_update_rate=1e-3, tie_word_embeddings=False, max_position_embeddings=1024,
        extra={"linear_backend": "seg_la"}, **kw)
    ec = EngineConfig(model=cfg, dummy_load=True, seed=9, optimizer=OptimizerConfig(lr=1e-4),
                      runtime=RuntimeConfig(max_model_len=256, max_prefill_tokens=64, activation_checkpointing=True),
                      max_running_seqs=4)
    worker = RankWorker(ec, dev)
    worker.loss_fn = loss_fns.grpo_loss_fn
    g = torch.Generator().manual_seed(10)
    prompts = [torch.randint(3, 2048, (n,), generator=g).tolist() for n in (40, 150, 9, 70, 21)]
    out = worker.rollout(prompts, SamplingParams(temperature=0.0), (), 8)
    agree = total = 0
    with torch.no_grad():
        for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
            ids = torch.tensor(p + toks, device=dev)
            meta = TrainMeta(build_varlen_meta([len(ids)], device=dev), False)
            h = worker.model(ids, torch.arange(len(ids), device=dev), meta).hidden_states
            lp_full = torch.log_softmax(worker.model.compute_logits(h).float(), -1)[len(p) - 1:-1]
            ref = lp_full.gather(-1, torch.tensor(toks, device=dev)[:, None]).squeeze(-1).cpu()
            err = (ref - torch.tensor(lps)).abs()   # a routing flip under bf16 noise moves single tokens
            assert err.max() < 0.3 and err.mean() < 0.04
            agree += sum(int(a == b) for a, b in zip(lp_full.argmax(-1).tolist(), toks))
            total += len(toks)
    assert agree >= 0.85 * total
    packs = []
    for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
        n = len(p) + len(toks)
        pm = torch.ones((1, n), dtype=torch.bool)
        pm[0, len(p):] = False
        lp = torch.zeros((1, n))
        lp[0, len(p):] = torch.tensor(lps)
        adv = torch.zeros((1, n))
        adv[0, len(p):] = 1.0
        packs.append(dict(input_ids=torch.tensor([p + toks]), lengths=torch.tensor([n]), prompt_mask=pm, logprobs=lp,
                          advantages=adv))
    stats = worker.train(packs)
    assert stats[-1]["stepped"] and stats[-1]["metrics"]["grad_norm"] > 0
    bias = worker.model.layers[1].mlp.gate.expert_bias
    assert float(bias.abs().max()) > 0 and abs(float(bias.mean())) < 1e-6      # the router bias moved, zero mean
    _lib.check_status()
