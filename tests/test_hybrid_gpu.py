"""Linear-attention kernels and the hybrid model on a B200 against their PyTorch references."""

from __future__ import annotations

import pytest
import torch

from areno_b200.ops import _lib, linear_attn as la

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.detach().float() - b.detach().float()).norm() / b.detach().float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("lens,C,K", [([70, 1, 300], 256, 4), ([5], 96, 3), ([2048], 1024, 4)])
def test_conv1d_silu_fwd_bwd(lens, C, K):
    torch.manual_seed(0)
    t = sum(lens)
    wide = torch.randn(t, C + 64, device="cuda").to(torch.bfloat16)
    x = wide[:, :C].detach().requires_grad_()            # strided rows, as in the fused projection output
    w = (torch.randn(C, K, device="cuda") * 0.5).requires_grad_()
    y = la.conv1d_silu(x, w, lens)
    xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    yr = la.conv1d_silu_reference(xr, wr, lens)
    assert _rel(y, yr) < 8e-3
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


def test_conv_history_and_decode():
    torch.manual_seed(1)
    C, K = 128, 4
    x = torch.randn(50, C, device="cuda").to(torch.bfloat16)
    w = torch.randn(C, K, device="cuda") * 0.5
    full = la.conv1d_silu_reference(x.float(), w, [50])
    cache = torch.zeros(4, C, K - 1, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    first = la.conv1d_silu(x[:2], w, [2])
    la.conv1d_update_hist(x[:2], i32([0, 2]), i32([3]), i32([1]), cache, K)       # shorter than the window
    second = la.conv1d_silu(x[2:30], w, [28], hist=cache[3:4].contiguous())
    la.conv1d_update_hist(x[2:30], i32([0, 28]), i32([3]), i32([0]), cache, K)
    assert _rel(torch.cat([first, second]), full[:30]) < 8e-3
    # decode continues slot 3; slot 1 is inactive and must keep its cache
    cache[1] = 7.0
    step = torch.zeros(4, C, device="cuda", dtype=torch.bfloat16)
    for r in range(30, 34):
        step[3] = x[r]
        y = la.conv1d_silu_decode(step, w, cache, i32([0, 0, 0, 1]))
        assert _rel(y[3], full[r]) < 1e-2
    assert bool((cache[1] == 7.0).all())


@pytest.mark.parametrize("hk,hv,dk,dv", [(2, 4, 128, 128), (4, 4, 64, 64), (1, 2, 32, 16)])
def test_gated_delta_rule_recurrent(hk, hv, dk, dv):
    torch.manual_seed(2)
    lens = [37, 5, 120]
    t = sum(lens)
    norm = lambda a: torch.nn.functional.normalize(a.float(), dim=-1).to(torch.bfloat16)
    q, k = norm(torch.randn(t, hk, dk, device="cuda")), norm(torch.randn(t, hk, dk, device="cuda"))
    v = torch.randn(t, hv, dv, device="cuda").to(torch.bfloat16)
    g, beta = -torch.rand(t, hv, device="cuda"), torch.rand(t, hv, device="cuda")
    cu = torch.tensor([0, 37, 42, 162], dtype=torch.int32, device="cuda")
    slots = torch.tensor([2, 0, 5], dtype=torch.int32, device="cuda")
    fresh = torch.tensor([1, 0, 1], dtype=torch.int32, device="cuda")
    cache = torch.randn(6, hv, dk, dv, device="cuda") * 0.1
    init = [torch.zeros_like(cache[0]), cache[0].clone(), torch.zeros_like(cache[0])]
    ref, finals = la.gated_delta_rule_reference(q, k, v, g, beta, lens, dk ** -0.5, init)
    out = la.gated_delta_rule_recurrent(q, k, v, g, beta, cu, dk ** -0.5, state_cache=cache, slots=slots, fresh=fresh)
    _lib.check_status()
    assert _rel(out, ref) < 1e-2
    for i, s in enumerate([2, 0, 5]):
        assert _rel(cache[s], finals[i]) < 1e-3
    # the chunk-parallel training path agrees as well (bf16 inputs)
    ch = la.gated_delta_rule_chunked(q, k, v, g, beta, lens, dk ** -0.5)
    ref0, _ = la.gated_delta_rule_reference(q, k, v, g, beta, lens, dk ** -0.5)
    assert _rel(ch, ref0) < 1e-2


@pytest.mark.parametrize("t,h,d", [(100, 4, 128), (7, 32, 64), (513, 2, 256)])
def test_rmsnorm_silu_gate(t, h, d):
    torch.manual_seed(3)
    x = torch.randn(t, h, d, device="cuda").to(torch.bfloat16).requires_grad_()
    wide = torch.randn(t, h * d + 32, device="cuda").to(torch.bfloat16)
    gate = wide[:, : h * d].unflatten(1, (h, d)).detach().requires_grad_()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).requires_grad_()
    y = la.rmsnorm_silu_gate(x, gate, w, 1e-6)
    xr, gr, wr = (a.detach().float().requires_grad_() for a in (x, gate, w))
    yr = la.rmsnorm_silu_gate_reference(xr, gr, wr, 1e-6)
    assert _rel(y, yr) < 8e-3
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(gate.grad, gr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


def test_hybrid_engine_matches_full_forward_and_trains():
    from areno_b200.api import loss_fns
    from areno_b200.engine.config import EngineConfig, ModelConfig, OptimizerConfig, RuntimeConfig
    from areno_b200.engine.inference import SamplingParams
    from areno_b200.engine.worker import RankWorker
    from areno_b200.models.dense import TrainMeta
    from areno_b200.ops.attention import build_varlen_meta
    from areno_b200.parallel.context import single_process_context

    dev = torch.device("cuda", 0)
    single_process_context(dev)
    cfg = ModelConfig(model_type="qwen3_5", vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=4,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, qk_norm=True, qkv_bias=False,
                      attn_output_gate=True, partial_rotary_factor=0.25, tie_word_embeddings=True,
                      layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                      linear_key_head_dim=64, linear_value_head_dim=64, linear_num_key_heads=2, linear_num_value_heads=4,
                      max_position_embeddings=1024)
    ec = EngineConfig(model=cfg, dummy_load=True, seed=5, optimizer=OptimizerConfig(lr=1e-4),
                      runtime=RuntimeConfig(max_model_len=256, max_prefill_tokens=64, activation_checkpointing=False),
                      max_running_seqs=4)
    worker = RankWorker(ec, dev)
    worker.loss_fn = loss_fns.grpo_loss_fn
    with torch.no_grad():
        for layer in worker.model._linear_layers():
            layer.attn.A_log.fill_(-1.0)
            layer.attn.dt_bias.fill_(0.5)
            layer.attn.norm_weight.fill_(1.0)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(3, 2048, (n,), generator=g).tolist() for n in (40, 150, 9, 70, 21)]
    out = worker.rollout(prompts, SamplingParams(temperature=0.0), (), 8)
    agree = total = 0
    with torch.no_grad():
        for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
            ids = torch.tensor(p + toks, device=dev)
            h = worker.model(ids, torch.arange(len(ids), device=dev), TrainMeta(build_varlen_meta([len(ids)], device=dev), False)).hidden_states
            lp_full = torch.log_softmax(worker.model.compute_logits(h).float(), -1)[len(p) - 1:-1]
            ref = lp_full.gather(-1, torch.tensor(toks, device=dev)[:, None]).squeeze(-1).cpu()
            assert (ref - torch.tensor(lps)).abs().max() < 0.08
            agree += sum(int(a == b) for a, b in zip(lp_full.argmax(-1).tolist(), toks))
            total += len(toks)
    assert agree >= 0.9 * total
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
    _lib.check_status()
