"""Hybrid (softmax + Gated DeltaNet) model on CPU: op references against each other, cached
inference (chunked prefill + decode) against a full forward, checkpoint round trip in the HF layout."""

from __future__ import annotations

import torch

from areno_b200.ops import linear_attn as la
from areno_b200.parallel.context import single_process_context

from .helpers import tiny_config


def hybrid_config(**kw):
    base = dict(model_type="qwen3_5", qk_norm=True, qkv_bias=False, attn_output_gate=True, partial_rotary_factor=0.5,
                layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"],
                num_hidden_layers=4, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16,
                linear_num_key_heads=2, linear_num_value_heads=4, tie_word_embeddings=True)
    base.update(kw)
    return tiny_config(**base)


def test_conv_reference_with_history_matches_one_pass():
    torch.manual_seed(0)
    x, w = torch.randn(40, 6), torch.randn(6, 4)
    full = la.conv1d_silu_reference(x, w, [40])
    # the same sequence in two chunks, carrying the last K-1 inputs over
    cache = torch.zeros(3, 6, 3)
    first = la.conv1d_silu_reference(x[:17], w, [17])
    la.conv1d_update_hist(x[:17], torch.tensor([0, 17], dtype=torch.int32), torch.tensor([2], dtype=torch.int32),
                          torch.tensor([1], dtype=torch.int32), cache, 4)
    second = la.conv1d_silu_reference(x[17:], w, [23], hist=cache[2:3])
    assert torch.allclose(torch.cat([first, second]), full, atol=1e-6)
    # decode steps continue from the cache (row i <-> slot i)
    la.conv1d_update_hist(x[17:39], torch.tensor([0, 22], dtype=torch.int32), torch.tensor([2], dtype=torch.int32),
                          torch.tensor([0], dtype=torch.int32), cache, 4)
    step_in = torch.zeros(3, 6)
    step_in[2] = x[39]
    y = la.conv1d_silu_decode(step_in, w, cache, torch.tensor([0, 0, 1], dtype=torch.int32))
    assert torch.allclose(y[2], full[39], atol=1e-6)
    # a chunk shorter than the window shifts older inputs in
    c2 = torch.zeros(1, 6, 3)
    zero = torch.tensor([0], dtype=torch.int32)
    la.conv1d_update_hist(x[:5], torch.tensor([0, 5], dtype=torch.int32), zero, torch.tensor([1], dtype=torch.int32), c2, 4)
    la.conv1d_update_hist(x[5:7], torch.tensor([0, 2], dtype=torch.int32), zero, zero, c2, 4)
    assert torch.allclose(c2[0].t(), x[4:7])


def test_chunked_delta_rule_matches_recurrence_and_is_differentiable():
    torch.manual_seed(1)
    t, hk, hv, dk, dv = 200, 2, 4, 16, 8
    lens = [77, 123]
    q = torch.nn.functional.normalize(torch.randn(t, hk, dk), dim=-1).requires_grad_()
    k = torch.nn.functional.normalize(torch.randn(t, hk, dk), dim=-1)
    v, g, beta = torch.randn(t, hv, dv), -torch.rand(t, hv), torch.rand(t, hv)
    ref, finals = la.gated_delta_rule_reference(q, k, v, g, beta, lens, dk ** -0.5)
    out = la.gated_delta_rule_chunked(q, k, v, g, beta, lens, dk ** -0.5, chunk=64)
    assert torch.allclose(out, ref, atol=1e-5)
    out.sum().backward()
    assert q.grad is not None and torch.isfinite(q.grad).all()
    # state hand-over: two halves with the carried state equal one pass
    a, fa = la.gated_delta_rule_reference(q[:40], k[:40], v[:40], g[:40], beta[:40], [40], dk ** -0.5)
    b, _ = la.gated_delta_rule_reference(q[40:77], k[40:77], v[40:77], g[40:77], beta[40:77], [37], dk ** -0.5, fa)
    assert torch.allclose(torch.cat([a, b]), ref[:77], atol=1e-5)


def test_cached_inference_matches_full_forward():
    from areno_b200.engine.inference import InferenceEngine, SamplingParams
    from areno_b200.models.dense import TrainMeta, init_weights
    from areno_b200.models.hybrid import HybridCausalLM
    from areno_b200.ops.attention import build_varlen_meta

    single_process_context()
    cfg = hybrid_config()
    model = HybridCausalLM(cfg)
    init_weights(model, 0)
    with torch.no_grad():
        for layer in model._linear_layers():
            layer.attn.A_log.fill_(-1.0)
            layer.attn.dt_bias.fill_(0.5)
    eng = InferenceEngine(model, 512, "cpu", max_slots=3, max_model_len=192, max_prefill_tokens=32)
    g = torch.Generator().manual_seed(3)
    # 5 prompts through 3 slots (slot reuse -> state reset), one longer than the prefill budget (chunked)
    prompts = [torch.randint(3, 512, (n,), generator=g).tolist() for n in (20, 70, 9, 33, 5)]
    out = eng.generate(prompts, SamplingParams(temperature=0.0), (), 6)
    with torch.no_grad():
        for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
            ids = torch.tensor(p + toks)
            h = model(ids, torch.arange(len(ids)), TrainMeta(build_varlen_meta([len(ids)]), False)).hidden_states
            logits = model.compute_logits(h).float()
            assert logits.argmax(-1)[len(p) - 1:-1].tolist() == toks
            ref = torch.log_softmax(logits, -1)[len(p) - 1:-1].gather(-1, torch.tensor(toks)[:, None]).squeeze(-1)
            assert torch.allclose(ref, torch.tensor(lps), atol=2e-3)


def test_checkpoint_round_trip_in_hf_layout(tmp_path):
    from areno_b200.engine.checkpoint import SafetensorsIndex
    from areno_b200.models import registry

    single_process_context()
    for name, prefix in (("qwen3_5", "model"), ("minicpmv46", "model.language_model")):
        adapter = registry.get_adapter(name)
        cfg = hybrid_config(model_type=name, checkpoint_prefix=prefix)
        model = adapter.build(cfg)
        adapter.init_random(model, 4)
        path = str(tmp_path / name)
        adapter.save_weights(model, path, cfg)
        index = SafetensorsIndex(path)
        q = index.get(f"{prefix}.layers.1.self_attn.q_proj.weight")
        assert q.shape[0] == 2 * cfg.num_attention_heads * cfg.head_dim       # queries interleaved with gates
        assert f"{prefix}.layers.0.linear_attn.in_proj_qkv.weight" in index
        assert tuple(index.shape(f"{prefix}.layers.0.linear_attn.conv1d.weight")) == (2 * 32 + 64, 1, 4)
        found, cfg2 = registry.config_from_pretrained(path)
        assert found.name == name and list(cfg2.layer_types) == list(cfg.layer_types)
        cfg2.dtype = torch.float32
        model2 = adapter.build(cfg2)
        adapter.load_weights(model2, path, cfg2)
        for (n1, p1), (n2, p2) in zip(model.named_parameters(), model2.named_parameters()):
            assert n1 == n2 and torch.equal(p1, p2), n1


def test_qwen35_moe_round_trip_and_step(tmp_path):
    from areno_b200.engine.checkpoint import SafetensorsIndex
    from areno_b200.models import registry
    from areno_b200.models.moe import SparseMoeBlock

    single_process_context()
    adapter = registry.get_adapter("qwen3_5_moe")
    cfg = hybrid_config(model_type="qwen3_5_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                        shared_expert_intermediate_size=48, norm_topk_prob=True, extra={"shared_expert_gate": True})
    model = adapter.build(cfg)
    adapter.init_random(model, 2)
    assert all(isinstance(layer.mlp, SparseMoeBlock) and layer.mlp.shared_gate is not None for layer in model.layers)
    path = str(tmp_path / "q35moe")
    adapter.save_weights(model, path, cfg)
    index = SafetensorsIndex(path)
    assert tuple(index.shape("model.layers.0.mlp.experts.gate_up_proj")) == (4, 64, 128)
    assert tuple(index.shape("model.layers.0.mlp.shared_expert_gate.weight")) == (1, 128)
    found, cfg2 = registry.config_from_pretrained(path)
    assert found.name == "qwen3_5_moe" and cfg2.num_experts == 4 and cfg2.shared_expert_intermediate_size == 48
    cfg2.dtype = torch.float32
    model2 = adapter.build(cfg2)
    adapter.load_weights(model2, path, cfg2)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), model2.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2), n1
    from areno_b200.models.dense import TrainMeta
    from areno_b200.ops.attention import build_varlen_meta

    ids = torch.randint(3, 512, (30,))
    h = model2(ids, torch.arange(30), TrainMeta(build_varlen_meta([30]), False)).hidden_states
    h.float().pow(2).mean().backward()
    assert model2.layers[0].mlp.shared_gate.grad is not None and model2.layers[0].mlp.router.weight.grad is not None
