"""Gemma-4 text model on CPU: cached inference (sliding window, KV-shared tail layers, PLE, MoE branch)
against a full forward, gradients reach every parameter, checkpoint round trip in the HF layout."""

from __future__ import annotations

import torch

from areno_b200.parallel.context import single_process_context

from .helpers import tiny_config


def gemma_config(**kw):
    base = dict(
        model_type="gemma4", num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=1, head_dim=32,
        swa_head_dim=16, swa_num_key_value_heads=2, qk_norm=True, v_norm=True, qkv_bias=False, hidden_act="gelu_tanh",
        layer_types=("sliding_attention", "sliding_attention", "full_attention", "sliding_attention", "full_attention",
                     "sliding_attention"),
        sliding_window=8, num_kv_shared_layers=2, use_double_wide_mlp=True, hidden_size_per_layer_input=16,
        vocab_size_per_layer_input=300, attention_softmax_scale=1.0, final_logit_softcapping=30.0, tie_word_embeddings=True,
        rope_parameters={"full_attention": {"rope_theta": 1e6, "partial_rotary_factor": 0.25},
                         "sliding_attention": {"rope_theta": 1e4}},
        enable_moe_block=True, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=True)
    base.update(kw)
    return tiny_config(**base)


def _model(cfg, seed=0):
    from areno_b200.models.dense import init_weights
    from areno_b200.models.gemma4 import Gemma4CausalLM

    single_process_context()
    model = Gemma4CausalLM(cfg)
    init_weights(model, seed)
    with torch.no_grad():
        for layer in model.layers:
            layer.layer_scalar.fill_(0.9)
            if layer.router is not None:
                layer.router.scale.fill_(1.0)
                layer.moe.per_expert_scale.fill_(1.0)
    return model


def test_structure():
    from areno_b200.models.gemma4 import kv_source_layer

    cfg = gemma_config()
    model = _model(cfg)
    assert [kv_source_layer(cfg, i) for i in range(6)] == [None, None, None, None, 2, 3]
    a_slide, a_full = model.layers[0].attn, model.layers[2].attn
    assert (a_slide.d, a_slide.hkv, a_slide.window) == (16, 2, 8) and (a_full.d, a_full.hkv, a_full.window) == (32, 1, 0)
    assert a_full.inv_freq.shape == (16,) and int((a_full.inv_freq > 0).sum()) == 4      # quarter of the head rotates
    assert model.layers[4].mlp.gate_up.weight.shape[0] == 2 * 2 * cfg.intermediate_size   # double-wide tail MLP
    assert model.layers[0].mlp.gate_up.weight.shape[0] == 2 * cfg.intermediate_size


def test_cached_inference_matches_full_forward_and_grads_flow(monkeypatch):
    from areno_b200.engine.inference import InferenceEngine, SamplingParams
    from areno_b200.models.dense import TrainMeta
    from areno_b200.ops import paged_attention as pa
    from areno_b200.ops.attention import build_varlen_meta

    def fp32_pages(num_pages, kv_heads, head_dim, device, fp8=False):   # bf16 pages would hide small errors
        shape = (num_pages, kv_heads, pa.PAGE, head_dim)
        return torch.zeros(shape, device=device), torch.zeros(shape, device=device), None, None

    monkeypatch.setattr(pa, "alloc_kv_cache", fp32_pages)

    cfg = gemma_config()
    model = _model(cfg, 1)
    eng = InferenceEngine(model, 512, "cpu", max_slots=3, max_model_len=128, max_prefill_tokens=24)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, 512, (n,), generator=g).tolist() for n in (15, 40, 6, 22)]   # 40 > budget: chunked
    out = eng.generate(prompts, SamplingParams(temperature=0.0), (), 12)
    with torch.no_grad():
        for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
            ids = torch.tensor(p + toks)
            h = model(ids, torch.arange(len(ids)), TrainMeta(build_varlen_meta([len(ids)]), False)).hidden_states
            logits = model.compute_logits(h).float()
            assert float(logits.abs().max()) <= 30.0 + 1e-4                      # soft cap
            assert logits.argmax(-1)[len(p) - 1:-1].tolist() == toks
            ref = torch.log_softmax(logits, -1)[len(p) - 1:-1].gather(-1, torch.tensor(toks)[:, None]).squeeze(-1)
            assert torch.allclose(ref, torch.tensor(lps), atol=1e-4)
    ids = torch.randint(3, 512, (50,), generator=g)
    h = model(ids, torch.arange(50), TrainMeta(build_varlen_meta([20, 30]), True)).hidden_states
    model.compute_logits(h).float().logsumexp(-1).mean().backward()
    missing = [n for n, p in model.named_parameters() if p.grad is None]
    assert missing == ["layers.4.attn.k_norm.weight", "layers.5.attn.k_norm.weight"], missing   # keys come from the source layer
    # KV-shared layers never use their own k / v rows: the gradient there is exactly zero
    a = model.layers[4].attn
    assert float(model.layers[4].attn.qkv.weight.grad[a.hq * a.d:].abs().max()) == 0.0
    assert float(model.layers[4].attn.qkv.weight.grad[: a.hq * a.d].abs().max()) > 0.0


def test_checkpoint_round_trip(tmp_path):
    from areno_b200.engine.checkpoint import SafetensorsIndex
    from areno_b200.models import registry

    for prefix in ("model", "model.language_model"):
        cfg = gemma_config(checkpoint_prefix=prefix)
        model = _model(cfg, 3)
        adapter = registry.get_adapter("gemma4")
        path = str(tmp_path / prefix.replace(".", "_"))
        adapter.save_weights(model, path, cfg)
        index = SafetensorsIndex(path)
        assert f"{prefix}.layers.0.experts.gate_up_proj" in index and f"{prefix}.layers.5.layer_scalar" in index
        assert tuple(index.shape(f"{prefix}.embed_tokens_per_layer.weight")) == (300, 6 * 16)
        found, cfg2 = registry.config_from_pretrained(path)
        assert found.name == "gemma4" and cfg2.checkpoint_prefix == prefix and cfg2.num_kv_shared_layers == 2
        assert cfg2.swa_head_dim == 16 and cfg2.head_dim == 32 and cfg2.enable_moe_block and cfg2.num_experts == 4
        cfg2.dtype = torch.float32
        model2 = adapter.build(cfg2)
        adapter.load_weights(model2, path, cfg2)
        for (n1, p1), (n2, p2) in zip(model.state_dict().items(), model2.state_dict().items()):
            rows = 300 if n1 == "embed_per_layer.weight" else p1.shape[0]   # rows past the vocabulary are padding
            assert n1 == n2 and torch.equal(p1[:rows], p2[:rows]), n1
