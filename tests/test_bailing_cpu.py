"""Bailing-MoE-Linear model on CPU: layer schedule and slopes, decayed linear attention and the gated group
norm against closed forms, router bias update, cached inference against the full forward for both softmax
variants (grouped-query and latent attention), gradients, checkpoint round trip."""

from __future__ import annotations

import pytest
import torch

from areno_b200.ops import linear_attn as la
from areno_b200.parallel.context import single_process_context

from .helpers import tiny_config


def bailing_config(mla: bool = False, **kw):
    base = dict(
        model_type="bailing_moe_linear_v2", num_hidden_layers=5, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
        qk_norm=True, qkv_bias=False, use_bias=False, layer_group_size=2, partial_rotary_factor=0.5, num_experts=8,
        num_experts_per_tok=2, n_group=2, topk_group=1, routed_scaling_factor=2.5, first_k_dense_replace=1,
        moe_intermediate_size=32, num_shared_experts=1, group_norm_size=4, qk_nope_head_dim=16, qk_rope_head_dim=16,
        v_head_dim=32, moe_router_bias_update_rate=1e-3, tie_word_embeddings=False, extra={"linear_backend": "seg_la"})
    if mla:
        base.update(kv_lora_rank=24, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32)
    base.update(kw)
    return tiny_config(**base)


def _model(cfg, seed=0):
    from areno_b200.models.bailing import BailingCausalLM
    from areno_b200.models.dense import init_weights

    single_process_context()
    model = BailingCausalLM(cfg)
    init_weights(model, seed)
    return model


def test_layer_schedule_and_slopes():
    from areno_b200.models.bailing import build_slopes, is_softmax_layer

    cfg = bailing_config()
    assert [is_softmax_layer(cfg, i) for i in range(5)] == [False, True, False, True, True]   # the tail layer anchors
    s8 = build_slopes(8, 0, 4)
    assert torch.allclose(s8, torch.tensor([2.0 ** -(i + 1) for i in range(8)]) * (1 + 1e-5))
    s6 = build_slopes(6, 3, 4)          # non power of two: 4 geometric + 2 interleaved from the 8-table
    assert s6.shape == (6,) and torch.allclose(s6, torch.tensor([0.25, 0.0625, 0.015625, 0.00390625, 0.5, 0.125]) * 1e-5)
    model = _model(cfg)
    kinds = [layer.kind for layer in model.layers]
    assert kinds == ["linear_attention", "attention", "linear_attention", "attention", "attention"]
    assert type(model.layers[0].mlp).__name__ == "GatedMLP" and type(model.layers[1].mlp).__name__ == "BailingSparseMoeBlock"


def test_lightning_reference_matches_closed_form_and_state_handover():
    torch.manual_seed(0)
    t, h, d = 23, 3, 8
    q, k, v = (torch.randn(t, h, d) for _ in range(3))
    slope = torch.tensor([0.5, 0.1, 0.01])
    out, finals = la.lightning_attention_reference(q, k, v, slope, [t], 0.3)
    idx = torch.arange(t)
    decay = torch.exp(-slope[:, None, None] * (idx[:, None] - idx[None, :]).clamp(min=0)) * (idx[:, None] >= idx[None, :])
    ref = torch.einsum("hts,shd->thd", torch.einsum("thd,shd->hts", q, k) * decay, v) * 0.3
    assert torch.allclose(out, ref, atol=1e-5)
    a, fa = la.lightning_attention_reference(q[:10], k[:10], v[:10], slope, [10], 0.3)
    b, fb = la.lightning_attention_reference(q[10:], k[10:], v[10:], slope, [13], 0.3, fa)
    assert torch.allclose(torch.cat([a, b]), out, atol=1e-5) and torch.allclose(fb[0], finals[0], atol=1e-5)


def test_group_rmsnorm_sigmoid_gate_reference():
    torch.manual_seed(1)
    x, gate, w = torch.randn(5, 24), torch.randn(5, 24), torch.rand(3, 8) + 0.5
    y = la.group_rmsnorm_sigmoid_gate(x, gate, w, 1e-6)
    for g in range(3):
        xs = x[:, g * 8:(g + 1) * 8]
        ref = xs / xs.pow(2).mean(-1, keepdim=True).add(1e-6).sqrt() * w[g] * torch.sigmoid(gate[:, g * 8:(g + 1) * 8])
        assert torch.allclose(y[:, g * 8:(g + 1) * 8], ref, atol=1e-6)


def test_gate_routing_and_bias_update():
    from areno_b200.models.bailing import BailingGate

    single_process_context()
    cfg = bailing_config()
    gate = BailingGate(cfg, "cpu")
    torch.manual_seed(2)
    with torch.no_grad():
        gate.weight.copy_(torch.randn_like(gate.weight))
    x = torch.randn(64, cfg.hidden_size)
    w, ids = gate(x)
    assert ids.shape == (64, 2) and torch.allclose(w.sum(-1), torch.full((64,), 2.5), atol=1e-5)   # renormalised x scaling
    assert bool(((ids[:, 0] // 4) == (ids[:, 1] // 4)).all())            # one group of four experts per token
    assert float(gate.tokens_per_expert.sum()) == 128.0
    counts = gate.tokens_per_expert.clone()
    gate.finalize_expert_bias(None)
    expect = torch.sign(counts.mean() - counts) * 1e-3
    assert torch.allclose(gate.expert_bias, expect - expect.mean(), atol=1e-9) and float(gate.tokens_per_expert.sum()) == 0.0
    with torch.no_grad():
        gate(x)
    assert float(gate.tokens_per_expert.sum()) == 0.0                    # evaluation does not count load


@pytest.mark.parametrize("mla", [False, True])
def test_cached_inference_matches_full_forward_and_grads_flow(mla, monkeypatch):
    from areno_b200.engine.inference import InferenceEngine, SamplingParams
    from areno_b200.models.dense import TrainMeta
    from areno_b200.ops import paged_attention as pa
    from areno_b200.ops.attention import build_varlen_meta

    def fp32_pages(num_pages, kv_heads, head_dim, device, fp8=False):
        shape = (num_pages, kv_heads, pa.PAGE, head_dim)
        return torch.zeros(shape, device=device), torch.zeros(shape, device=device), None, None

    monkeypatch.setattr(pa, "alloc_kv_cache", fp32_pages)
    cfg = bailing_config(mla)
    model = _model(cfg, 3)
    eng = InferenceEngine(model, 512, "cpu", max_slots=3, max_model_len=128, max_prefill_tokens=24)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, 512, (n,), generator=g).tolist() for n in (15, 40, 6, 22)]   # 40 > budget: chunked
    out = eng.generate(prompts, SamplingParams(temperature=0.0), (), 10)
    with torch.no_grad():
        for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
            ids = torch.tensor(p + toks)
            h = model(ids, torch.arange(len(ids)), TrainMeta(build_varlen_meta([len(ids)]), False)).hidden_states
            logits = model.compute_logits(h).float()
            assert logits.argmax(-1)[len(p) - 1:-1].tolist() == toks
            ref = torch.log_softmax(logits, -1)[len(p) - 1:-1].gather(-1, torch.tensor(toks)[:, None]).squeeze(-1)
            assert torch.allclose(ref, torch.tensor(lps), atol=1e-4)
    ids = torch.randint(3, 512, (50,), generator=g)
    h = model(ids, torch.arange(50), TrainMeta(build_varlen_meta([20, 30]), True)).hidden_states
    model.compute_logits(h).float().logsumexp(-1).mean().backward()
    missing = [n for n, p in model.named_parameters() if p.grad is None]
    assert all(n.endswith("mlp.gate.weight") for n in missing), missing     # routing weights carry no gradient
    model.finalize_router_expert_bias(None, None)


def test_checkpoint_round_trip_and_prefix_alias(tmp_path):
    from safetensors.torch import load_file, save_file

    from areno_b200.models import registry

    for mla in (False, True):
        cfg = bailing_config(mla)
        model = _model(cfg, 5)
        with torch.no_grad():
            model.layers[1].mlp.gate.expert_bias.copy_(torch.linspace(-1, 1, 8))
        adapter = registry.get_adapter("bailing_moe_linear_v2")
        path = str(tmp_path / f"ckpt{int(mla)}")
        adapter.save_weights(model, path, cfg)
        tensors = load_file(f"{path}/model.safetensors")
        assert "model.word_embeddings.weight" in tensors and "model.layers.1.mlp.experts.7.down_proj.weight" in tensors
        assert "model.layers.0.attention.g_norm.weight" in tensors and "model.layers.1.mlp.gate.expert_bias" in tensors
        assert ("model.layers.1.attention.kv_a_proj_with_mqa.weight" in tensors) == mla
        # rewrite with the other attention prefix: the loader accepts both
        save_file({k.replace(".attention.", ".self_attn."): v for k, v in tensors.items()},
                  f"{path}/model.safetensors", metadata={"format": "pt"})
        import json
        with open(f"{path}/model.safetensors.index.json") as f:
            idx = json.load(f)
        idx["weight_map"] = {k.replace(".attention.", ".self_attn."): v for k, v in idx["weight_map"].items()}
        with open(f"{path}/model.safetensors.index.json", "w") as f:
            json.dump(idx, f)
        found, cfg2 = registry.config_from_pretrained(path)
        assert found.name == "bailing_moe_linear_v2" and cfg2.layer_group_size == 2 and cfg2.n_group == 2
        assert cfg2.kv_lora_rank == (24 if mla else None) and cfg2.num_shared_experts == 1
        cfg2.dtype = torch.float32
        model2 = adapter.build(cfg2)
        adapter.load_weights(model2, path, cfg2)
        for (n1, p1), (n2, p2) in zip(model.state_dict().items(), model2.state_dict().items()):
            assert n1 == n2 and torch.equal(p1, p2), n1
        assert torch.equal(model2.layers[1].mlp.gate.expert_bias, torch.linspace(-1, 1, 8))
