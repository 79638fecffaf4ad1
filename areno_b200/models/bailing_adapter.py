"""Adapter for Bailing-MoE-Linear-V2 / V2.5 checkpoints (``architectures`` contains
``BailingMoeV2_5ForCausalLM`` or ``model_type == "bailing_moe_linear"``; reference:
``areno/models/bailing/model.py:1236-1358`` and ``checkpoint.py``).  Tensor names follow the HF layout:
``model.word_embeddings``, fused ``attention.query_key_value`` (or the latent-attention projections),
``attention.dense``, ``attention.g_proj`` / ``g_norm`` on linear layers, ``mlp.gate.weight`` /
``mlp.gate.expert_bias``, one ``mlp.experts.{e}.{gate,up,down}_proj`` triple per routed expert and
``mlp.shared_experts``.  Both ``attention`` and ``self_attn`` are accepted as the attention prefix on load.
At tensor-parallel size > 1 every rank cuts its heads / features / experts out of the HF tensors on load and the
shards are gathered inside the TP group on save (TP rank 0 writes)."""

from __future__ import annotations

import json
import os
from typing import Any

import torch

from ..engine.config import ModelConfig, parse_dtype
from .bailing import BailingCausalLM, BailingLinearAttention, BailingMLAttention, BailingSparseMoeBlock
from .base import ModelAdapter


def _bool(value: Any, default: bool) -> bool:
    if value is None:
        return default
    if isinstance(value, str):
        return value.strip().lower() in ("1", "true", "yes", "on")
    return bool(value)


def _dtype(name: Any, default=torch.bfloat16):
    return parse_dtype(name, default)


def _tensor_plan(model: BailingCausalLM, cfg: ModelConfig):
    """Yield ``(hf_key, getter, setter, kind)`` for every tensor; attention keys carry ``{attn}`` for the prefix alias.
    ``getter`` / ``setter`` address this rank's part, ``kind`` says how it sits in the full tensor (the kinds of
    ``gemma4_adapter._local_part``; ``expert`` marks one routed expert's matrix, whose key carries the global index)."""

    def whole(t):
        return (lambda: t.detach()), (lambda v: t.copy_(v.reshape(t.shape).to(t.dtype)))

    def rows(t, lo, hi):
        return (lambda: t.detach()[lo:hi]), (lambda v: t[lo:hi].copy_(v.to(t.dtype)))

    def expert(t, e, lo, hi):
        return (lambda: t.detach()[e, lo:hi]), (lambda v: t[e, lo:hi].copy_(v.to(t.dtype)))

    yield ("model.word_embeddings.weight", *whole(model.embed.weight), f"vocab:{cfg.vocab_size}")
    yield ("model.norm.weight", *whole(model.norm.weight), "rep")
    if not cfg.tie_word_embeddings:
        yield ("lm_head.weight", *whole(model.lm_head.weight), f"vocab:{cfg.vocab_size}")
    for i, layer in enumerate(model.layers):
        lp = f"model.layers.{i}"
        yield (f"{lp}.input_layernorm.weight", *whole(layer.input_norm.weight), "rep")
        yield (f"{lp}.post_attention_layernorm.weight", *whole(layer.post_norm.weight), "rep")
        a, ap = layer.attn, f"{lp}.{{attn}}"
        if isinstance(a, BailingMLAttention):
            yield (f"{ap}.q_proj.weight", *whole(a.q_proj.weight), "rows")
            yield (f"{ap}.kv_a_proj_with_mqa.weight", *whole(a.kv_a), "rep")
            yield (f"{ap}.kv_a_layernorm.weight", *whole(a.kv_a_norm.weight), "rep")
            yield (f"{ap}.kv_b_proj.weight", *whole(a.kv_b.weight), "rows")
            out = a.o
        else:
            if isinstance(a, BailingLinearAttention):
                fused = "parts:3"
            else:
                fused = f"qkv:{a.hq * a.d}:{a.hkv * a.d}:{a.qkv.kv_rep}"
            yield (f"{ap}.query_key_value.weight", *whole(a.qkv.weight), fused)
            if a.qkv.bias is not None:
                yield (f"{ap}.query_key_value.bias", *whole(a.qkv.bias), fused)
            if a.q_norm is not None:
                yield (f"{ap}.query_layernorm.weight", *whole(a.q_norm.weight), "rep")
                yield (f"{ap}.key_layernorm.weight", *whole(a.k_norm.weight), "rep")
            if isinstance(a, BailingLinearAttention):
                yield (f"{ap}.g_proj.weight", *whole(a.g_proj.weight), "rows")
                yield (f"{ap}.g_norm.weight", *whole(a.g_norm_weight), "rows")
                out = a.out_proj
            else:
                out = a.o
        yield (f"{ap}.dense.weight", *whole(out.weight), "cols")
        if out.bias is not None:
            yield (f"{ap}.dense.bias", *whole(out.bias), "rep")
        mlp = layer.mlp
        if isinstance(mlp, BailingSparseMoeBlock):
            yield (f"{lp}.mlp.gate.weight", *whole(mlp.gate.weight), "rep")
            yield (f"{lp}.mlp.gate.expert_bias", *whole(mlp.gate.expert_bias), "rep")
            inter = cfg.moe_intermediate_size
            for e in range(mlp.experts.e_local):
                ge = "{expert" + str(e) + "}"      # filled in with the global expert index of the rank that owns it
                yield (f"{lp}.mlp.experts.{ge}.gate_proj.weight", *expert(mlp.experts.gate_up, e, 0, inter), f"expert:{e}")
                yield (f"{lp}.mlp.experts.{ge}.up_proj.weight", *expert(mlp.experts.gate_up, e, inter, 2 * inter), f"expert:{e}")
                yield (f"{lp}.mlp.experts.{ge}.down_proj.weight", *expert(mlp.experts.down, e, 0, cfg.hidden_size), f"expert:{e}")
            dense, dp = mlp.shared, f"{lp}.mlp.shared_experts"
        else:
            dense, dp = mlp, f"{lp}.mlp"
        if dense is not None:
            half = dense.gate_up.weight.shape[0] // 2
            yield (f"{dp}.gate_proj.weight", *rows(dense.gate_up.weight, 0, half), "rows")
            yield (f"{dp}.up_proj.weight", *rows(dense.gate_up.weight, half, 2 * half), "rows")
            yield (f"{dp}.down_proj.weight", *whole(dense.down.weight), "cols")


def _expert_key(key: str, local_e: int, e_local: int, rank: int) -> str:
    return key.replace("{expert" + str(local_e) + "}", str(rank * e_local + local_e))


_OPTIONAL_SUFFIXES = ("mlp.gate.expert_bias",)


class BailingMoeLinearV2Adapter(ModelAdapter):
    name = "bailing_moe_linear_v2"

    def match_hf_config(self, hf):
        return "BailingMoeV2_5ForCausalLM" in (hf.get("architectures") or []) or \
            str(hf.get("model_type", "")).lower() in ("bailing_moe_linear", self.name)

    def config_from_hf(self, hf) -> ModelConfig:
        heads = int(hf["num_attention_heads"])
        head_dim = int(hf.get("head_dim", int(hf["hidden_size"]) // heads))
        rotary_dim = int(hf.get("rotary_dim", hf.get("qk_rope_head_dim", head_dim)))
        moe_inter = int(hf.get("moe_intermediate_size", hf.get("intermediate_size", 0)))
        shared_size, shared_n = hf.get("moe_shared_expert_intermediate_size"), hf.get("num_shared_experts")
        if shared_size is not None and shared_n is None:
            shared_n = max(1, int(shared_size) // max(1, moe_inter))
        backend = str(hf.get("linear_backend", "seg_la")).lower()
        score = str(hf.get("score_function", hf.get("scoring_func", hf.get("moe_router_score_function", "sigmoid")))).lower()
        method = str(hf.get("topk_method", "noaux_tc")).lower()
        bias_on = _bool(hf.get("moe_router_enable_expert_bias"), True)
        renorm = _bool(hf.get("norm_topk_prob"), True)
        if score != "sigmoid":
            raise ValueError(f"BailingMoeLinearV2 only supports score_function='sigmoid', got {score!r}")
        if not bias_on:
            raise ValueError("BailingMoeLinearV2 requires moe_router_enable_expert_bias=True (biased grouped top-k)")
        if not renorm:
            raise ValueError("BailingMoeLinearV2 requires norm_topk_prob=True")
        if method not in ("noaux_tc", "group_limited_greedy"):
            raise ValueError(f"unsupported BailingMoeLinearV2 topk_method={method!r}")
        experts = hf.get("num_experts", hf.get("n_routed_experts"))
        return ModelConfig(
            model_type=self.name, vocab_size=int(hf["vocab_size"]), hidden_size=int(hf["hidden_size"]),
            intermediate_size=int(hf["intermediate_size"]), num_hidden_layers=int(hf["num_hidden_layers"]),
            num_attention_heads=heads, num_key_value_heads=int(hf.get("num_key_value_heads", heads)), head_dim=head_dim,
            rms_norm_eps=float(hf.get("rms_norm_eps", 1e-6)), rope_theta=float(hf.get("rope_theta", hf.get("rotary_base", 10000.0))),
            max_position_embeddings=int(hf.get("max_position_embeddings", 4096)),
            tie_word_embeddings=_bool(hf.get("tie_word_embeddings"), False),
            qkv_bias=_bool(hf.get("use_qkv_bias", hf.get("qkv_bias")), False), qk_norm=_bool(hf.get("use_qk_norm"), True),
            dtype=_dtype(hf.get("torch_dtype") or hf.get("dtype")), hidden_act=str(hf.get("hidden_act", "silu")),
            use_bias=_bool(hf.get("use_bias"), False), layer_group_size=int(hf.get("layer_group_size", 1)),
            partial_rotary_factor=float(hf.get("partial_rotary_factor", rotary_dim / head_dim)),
            num_experts=int(experts) if experts is not None else None,
            num_experts_per_tok=int(hf.get("num_experts_per_tok", hf.get("moe_router_topk", 1))),
            n_group=int(hf.get("n_group", hf.get("moe_router_num_groups", 1))),
            topk_group=int(hf.get("topk_group", hf.get("moe_router_group_topk", 1))),
            routed_scaling_factor=float(hf.get("routed_scaling_factor", hf.get("moe_router_topk_scaling_factor", 1.0))),
            first_k_dense_replace=int(hf.get("first_k_dense_replace", 0)), moe_intermediate_size=moe_inter,
            num_shared_experts=int(shared_n) if shared_n is not None else None, moe_router_enable_expert_bias=bias_on,
            norm_topk_prob=renorm, moe_router_dtype=_dtype(hf.get("moe_router_dtype") or "fp32", torch.float32),
            score_function=score, topk_method=method,
            group_norm_size=int(hf.get("group_norm_size", hf.get("linear_attn_norm_group_size", hf.get("head_dim", 128)))),
            qk_nope_head_dim=int(hf.get("qk_nope_head_dim", head_dim)), qk_rope_head_dim=int(hf.get("qk_rope_head_dim", rotary_dim)),
            v_head_dim=int(hf.get("v_head_dim", head_dim)), kv_lora_rank=hf.get("kv_lora_rank"),
            linear_scale=backend == "minimax", linear_silu=_bool(hf.get("use_linear_silu", hf.get("linear_silu")), False),
            sequence_parallel=_bool(hf.get("sequence_parallel"), True),
            moe_router_bias_update_rate=float(hf.get("moe_router_bias_update_rate", 0.0)),
            extra={"linear_backend": backend, "num_nextn_predict_layers": int(hf.get("num_nextn_predict_layers", 0)),
                   "mtp_loss_scaling_factor": float(hf.get("mtp_loss_scaling_factor", 0.0))})

    def build(self, config, device="cpu"):
        return BailingCausalLM(config, device=device)

    @torch.no_grad()
    def load_weights(self, model, path, config):
        from ..engine.checkpoint import SafetensorsIndex, logger
        from ..parallel.context import get_context

        from .gemma4_adapter import _local_part

        ctx = get_context()
        tp, rank = ctx.tp_size, ctx.tp_rank
        e_local = int(config.num_experts) // tp if config.num_experts else 0
        index = SafetensorsIndex(path)
        used = 0
        for n_seen, (key, _get, put, kind) in enumerate(_tensor_plan(model, config)):
            if kind.startswith("expert:"):
                key = _expert_key(key, int(kind[7:]), e_local, rank)
                kind = "rep"
            found = next((k for k in (key.format(attn="attention"), key.format(attn="self_attn")) if k in index), None)
            if found is None and key.endswith("query_key_value.weight"):
                alt = key.replace("query_key_value", "qkv")
                found = next((k for k in (alt.format(attn="attention"), alt.format(attn="self_attn")) if k in index), None)
            if found is None:
                if key.endswith(_OPTIONAL_SUFFIXES):
                    continue
                raise KeyError(f"checkpoint is missing {key.format(attn='attention')}")
            put(_local_part(index.get(found), tuple(_get().shape), kind, tp, rank))
            used += 1
            if n_seen % 256 == 255:
                index.drop()
        index.drop()
        logger.info("checkpoint loaded path=%s tensors=%d", path, used)

    @torch.no_grad()
    def save_weights(self, model, path, config, source_path=None):
        from safetensors.torch import save_file

        from ..engine.checkpoint import _passthrough_untouched, copy_assets
        from ..parallel.context import get_context

        import torch.distributed as dist

        from .gemma4_adapter import _full_tensor
        from .hybrid_adapters import _full

        ctx = get_context()
        if ctx.dp_rank != 0:
            if ctx.world_size > 1:
                dist.barrier()
            return
        os.makedirs(path, exist_ok=True)
        tp = ctx.tp_size
        writer = ctx.tp_rank == 0          # every rank of the TP group takes part in the gathers, one writes
        e_local = int(config.num_experts) // tp if config.num_experts else 0
        out = {}
        for key, get, _put, kind in _tensor_plan(model, config):
            if kind.startswith("expert:"):
                local = get().contiguous()
                stacked = _full(local.unsqueeze(0), 0)             # [tp, ...]: the same local expert slot of every rank
                if writer:
                    for r in range(tp):
                        name = _expert_key(key, int(kind[7:]), e_local, r).replace("{attn}", "attention")
                        out[name] = stacked[r].to("cpu", copy=True).contiguous()
                continue
            full = _full_tensor(get(), kind)
            if writer:
                out[key.replace("{attn}", "attention")] = full.to("cpu", copy=True).contiguous()
        if not writer:
            dist.barrier()
            return
        fname = "model.safetensors"
        save_file(out, os.path.join(path, fname), metadata={"format": "pt"})
        weight_map = {k: fname for k in out}
        total = sum(t.numel() * t.element_size() for t in out.values())
        if source_path and os.path.isdir(source_path):
            total += _passthrough_untouched(source_path, path, weight_map)
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total, "areno_checkpoint_writer": "distributed_tp"},
                       "weight_map": dict(sorted(weight_map.items()))}, f, indent=2)
        copy_assets(source_path, path, None)
        if not os.path.exists(os.path.join(path, "config.json")):
            with open(os.path.join(path, "config.json"), "w") as f:
                json.dump(self.hf_config(config), f, indent=2)
        if ctx.world_size > 1:
            dist.barrier()

    @staticmethod
    def hf_config(c: ModelConfig) -> dict[str, Any]:
        return {
            "architectures": ["BailingMoeV2_5ForCausalLM"], "model_type": "bailing_moe_linear", "vocab_size": c.vocab_size,
            "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size, "num_hidden_layers": c.num_hidden_layers,
            "num_attention_heads": c.num_attention_heads, "num_key_value_heads": c.num_key_value_heads, "head_dim": c.head_dim,
            "rms_norm_eps": c.rms_norm_eps, "rope_theta": c.rope_theta, "max_position_embeddings": c.max_position_embeddings,
            "tie_word_embeddings": c.tie_word_embeddings, "use_qkv_bias": c.qkv_bias, "use_qk_norm": c.qk_norm,
            "hidden_act": c.hidden_act, "use_bias": c.use_bias, "layer_group_size": c.layer_group_size,
            "partial_rotary_factor": c.partial_rotary_factor, "num_experts": c.num_experts,
            "num_experts_per_tok": c.num_experts_per_tok, "n_group": c.n_group, "topk_group": c.topk_group,
            "routed_scaling_factor": c.routed_scaling_factor, "first_k_dense_replace": c.first_k_dense_replace,
            "moe_intermediate_size": c.moe_intermediate_size, "num_shared_experts": c.num_shared_experts,
            "moe_router_enable_expert_bias": True, "norm_topk_prob": True, "score_function": "sigmoid",
            "topk_method": c.topk_method, "group_norm_size": c.group_norm_size, "qk_nope_head_dim": c.qk_nope_head_dim,
            "qk_rope_head_dim": c.qk_rope_head_dim, "v_head_dim": c.v_head_dim, "kv_lora_rank": c.kv_lora_rank,
            "linear_backend": (c.extra or {}).get("linear_backend", "seg_la"), "use_linear_silu": c.linear_silu,
            "moe_router_bias_update_rate": c.moe_router_bias_update_rate, "moe_router_dtype": "fp32",
            "torch_dtype": str(c.dtype).replace("torch.", ""),
        }


ADAPTERS = [BailingMoeLinearV2Adapter]
