"""Adapters of the hybrid (softmax + Gated DeltaNet) text models: ``qwen3_5`` and the text trunk of
``minicpmv4_6`` (reference: ``areno/models/qwen3_5/model.py:805-880``, ``checkpoint.py:36-100,560-675``;
``areno/models/minicpmv46/model.py:655-717``).

Checkpoint layout handled here: HF stores the attention output gate
interleaved with the queries in ``q_proj`` (``[heads, 2, head_dim]`` rows) and the linear-attention
input projections as four tensors (``in_proj_qkv``, ``in_proj_z``, ``in_proj_b``, ``in_proj_a``);
they are regrouped into this package's fused parameters on load and split again on save.  Tensors
outside the text trunk (vision tower, projector) pass through untouched when saving from a source
directory.  At tensor-parallel size > 1 every rank cuts its heads / features / experts out of the HF tensors on
load; on save the shards are gathered inside the TP group and TP rank 0 of the first data-parallel replica writes
one file in the same HF layout."""

from __future__ import annotations

import json
import os
from typing import Any

import torch

from ..engine.config import ModelConfig, parse_dtype
from .base import ModelAdapter
from .hybrid import GatedDeltaNet, HybridCausalLM


def _layer_types(n: int, interval: int) -> list[str]:
    return ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(n)]


def _text_config(hf: dict[str, Any], name: str, prefix: str) -> ModelConfig:
    text = hf.get("text_config") or hf
    rope = text.get("rope_parameters") or text.get("rope_scaling") or {}
    n = int(text["num_hidden_layers"])
    heads = int(text["num_attention_heads"])
    dtype = parse_dtype(text.get("torch_dtype") or text.get("dtype") or hf.get("torch_dtype") or hf.get("dtype"))
    return ModelConfig(
        model_type=name, checkpoint_prefix=prefix, vocab_size=int(text["vocab_size"]), hidden_size=int(text["hidden_size"]),
        intermediate_size=int(text["intermediate_size"]), num_hidden_layers=n, num_attention_heads=heads,
        num_key_value_heads=int(text.get("num_key_value_heads", heads)),
        head_dim=int(text.get("head_dim", int(text["hidden_size"]) // heads)),
        rms_norm_eps=float(text.get("rms_norm_eps", 1e-6)),
        rope_theta=float(rope.get("rope_theta", text.get("rope_theta", 10_000.0))),
        max_position_embeddings=int(text.get("max_position_embeddings", 262144)),
        tie_word_embeddings=bool(text.get("tie_word_embeddings", hf.get("tie_word_embeddings", True))),
        qkv_bias=bool(text.get("attention_bias", False)), qk_norm=True, dtype=dtype,
        hidden_act=str(text.get("hidden_act", "silu")),
        layer_types=list(text.get("layer_types") or _layer_types(n, int(text.get("full_attention_interval", 1)))),
        partial_rotary_factor=float(rope.get("partial_rotary_factor", text.get("partial_rotary_factor", 0.25))),
        attn_output_gate=bool(text.get("attn_output_gate", True)),
        linear_conv_kernel_dim=int(text.get("linear_conv_kernel_dim", 4)),
        linear_key_head_dim=int(text.get("linear_key_head_dim", 128)),
        linear_value_head_dim=int(text.get("linear_value_head_dim", 128)),
        linear_num_key_heads=int(text.get("linear_num_key_heads", 16)),
        linear_num_value_heads=int(text.get("linear_num_value_heads", 32)),
    )


def _hf_text_config(c: ModelConfig) -> dict[str, Any]:
    out = _hf_text_config_base(c)
    if c.num_experts:
        out.update(num_experts=c.num_experts, num_experts_per_tok=c.num_experts_per_tok,
                   moe_intermediate_size=c.moe_intermediate_size, norm_topk_prob=c.norm_topk_prob,
                   shared_expert_intermediate_size=c.shared_expert_intermediate_size)
    return out


def _hf_text_config_base(c: ModelConfig) -> dict[str, Any]:
    return {
        "model_type": c.model_type, "vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
        "intermediate_size": c.intermediate_size, "num_hidden_layers": c.num_hidden_layers,
        "num_attention_heads": c.num_attention_heads, "num_key_value_heads": c.num_key_value_heads, "head_dim": c.head_dim,
        "rms_norm_eps": c.rms_norm_eps, "rope_theta": c.rope_theta, "max_position_embeddings": c.max_position_embeddings,
        "tie_word_embeddings": c.tie_word_embeddings, "attention_bias": c.qkv_bias, "hidden_act": c.hidden_act,
        "torch_dtype": str(c.dtype).replace("torch.", ""), "layer_types": list(c.layer_types or []),
        "partial_rotary_factor": c.partial_rotary_factor, "attn_output_gate": c.attn_output_gate,
        "linear_conv_kernel_dim": c.linear_conv_kernel_dim, "linear_key_head_dim": c.linear_key_head_dim,
        "linear_value_head_dim": c.linear_value_head_dim, "linear_num_key_heads": c.linear_num_key_heads,
        "linear_num_value_heads": c.linear_num_value_heads,
    }


def _prefix_in(index, candidates: tuple[str, ...]) -> str:
    for p in candidates:
        if f"{p}.embed_tokens.weight" in index:
            return p
    raise KeyError(f"no embedding found under any of {candidates}")


def _tp():
    from ..parallel.context import get_context

    ctx = get_context()
    return ctx.tp_size, ctx.tp_rank


def _sh0(t: torch.Tensor) -> torch.Tensor:
    """This rank's equal share of dim 0."""
    tp, r = _tp()
    return t if tp == 1 else t.chunk(tp, 0)[r]


def _sh1(t: torch.Tensor) -> torch.Tensor:
    tp, r = _tp()
    return t if tp == 1 else t.chunk(tp, 1)[r]


def _full(t: torch.Tensor, dim: int = 0) -> torch.Tensor:
    """All TP shards of ``t`` concatenated along ``dim`` (on every rank of the group)."""
    from ..parallel.context import get_context

    ctx = get_context()
    if ctx.tp_size == 1:
        return t
    import torch.distributed as dist

    t = t.detach().contiguous()
    parts = [torch.empty_like(t) for _ in range(ctx.tp_size)]
    dist.all_gather(parts, t, group=ctx.tp_group)
    return torch.cat(parts, dim=dim)


def _full_kv(t: torch.Tensor, rep: int) -> torch.Tensor:
    """Gather K / V rows whose heads are replicated ``rep`` times over neighbouring ranks: keep one copy of each."""
    full = _full(t, 0)
    if rep <= 1:
        return full
    tp, _ = _tp()
    return full.view(tp // rep, rep, t.shape[0], *full.shape[1:])[:, 0].reshape(-1, *full.shape[1:])


def _load_dense_mlp(index, mlp, mp: str, put) -> None:
    put(mlp.gate_up.weight, torch.cat([_sh0(index.get(f"{mp}.gate_proj.weight")), _sh0(index.get(f"{mp}.up_proj.weight"))], 0))
    put(mlp.down.weight, _sh1(index.get(f"{mp}.down_proj.weight")))


def _load_mlp(index, mlp, mp: str, put) -> int:
    """Dense SwiGLU, or router + routed experts (packed ``experts.gate_up_proj`` / ``experts.down_proj`` or one
    tensor per expert) + optional shared expert with its sigmoid gate."""
    from .moe import SparseMoeBlock

    if not isinstance(mlp, SparseMoeBlock):
        _load_dense_mlp(index, mlp, mp, put)
        return 0
    gate_key = next(k for k in (f"{mp}.gate.weight", f"{mp}.gate", f"{mp}.router.weight") if k in index)
    put(mlp.router.weight, index.get(gate_key))
    ex = mlp.experts
    packed = next(((a, b) for a, b in ((f"{mp}.experts.gate_up_proj.weight", f"{mp}.experts.down_proj.weight"),
                                       (f"{mp}.experts.gate_up_proj", f"{mp}.experts.down_proj")) if a in index), None)
    if packed is not None:
        put(ex.gate_up, index.get(packed[0])[ex.e_lo: ex.e_lo + ex.e_local])
        put(ex.down, index.get(packed[1])[ex.e_lo: ex.e_lo + ex.e_local])
    else:
        for le in range(ex.e_local):
            e = ex.e_lo + le
            put(ex.gate_up[le], torch.cat([index.get(f"{mp}.experts.{e}.gate_proj.weight"),
                                           index.get(f"{mp}.experts.{e}.up_proj.weight")], 0))
            put(ex.down[le], index.get(f"{mp}.experts.{e}.down_proj.weight"))
    if mlp.shared is not None:
        _load_dense_mlp(index, mlp.shared, f"{mp}.shared_expert", put)
    if mlp.shared_gate is not None:
        put(mlp.shared_gate, index.get(f"{mp}.shared_expert_gate.weight").reshape(-1))
    return 0


def _save_mlp(out: dict, mlp, mp: str, cpu) -> None:
    from .moe import SparseMoeBlock

    def dense(m, prefix):
        inter = m.gate_up.weight.shape[0] // 2
        out[f"{prefix}.gate_proj.weight"] = cpu(_full(m.gate_up.weight[:inter], 0))
        out[f"{prefix}.up_proj.weight"] = cpu(_full(m.gate_up.weight[inter:], 0))
        out[f"{prefix}.down_proj.weight"] = cpu(_full(m.down.weight, 1))

    if not isinstance(mlp, SparseMoeBlock):
        dense(mlp, mp)
        return
    out[f"{mp}.gate.weight"] = cpu(mlp.router.weight)
    out[f"{mp}.experts.gate_up_proj"] = cpu(_full(mlp.experts.gate_up, 0))
    out[f"{mp}.experts.down_proj"] = cpu(_full(mlp.experts.down, 0))
    if mlp.shared is not None:
        dense(mlp.shared, f"{mp}.shared_expert")
    if mlp.shared_gate is not None:
        out[f"{mp}.shared_expert_gate.weight"] = cpu(mlp.shared_gate.reshape(1, -1))


class _HybridAdapter(ModelAdapter):
    prefixes: tuple[str, ...] = ("model", "model.language_model")

    def build(self, config, device="cpu"):
        return HybridCausalLM(config, device=device)

    # ------------------------------------------------------------------ load
    @torch.no_grad()
    def load_weights(self, model, path, config):
        from ..engine.checkpoint import Rule, SafetensorsIndex, load_rule, logger

        tp, rank = _tp()
        index = SafetensorsIndex(path)
        pre = _prefix_in(index, self.prefixes)
        used = 0

        def put(param, tensor):
            nonlocal used
            if tuple(param.shape) != tuple(tensor.shape):
                raise ValueError(f"shape mismatch: checkpoint {tuple(tensor.shape)} vs parameter {tuple(param.shape)}")
            param.copy_(tensor.to(param.dtype))
            used += 1

        def put_vocab(param, key):
            nonlocal used
            load_rule(index, param, Rule("", (key,), "vocab"), (key,))   # this rank's rows, zero padded
            used += 1

        put_vocab(model.embed.weight, f"{pre}.embed_tokens.weight")
        put(model.norm.weight, index.get(f"{pre}.norm.weight"))
        if not config.tie_word_embeddings:
            put_vocab(model.lm_head.weight, next(k for k in (f"{pre}.lm_head.weight", "lm_head.weight") if k in index))
        for i, layer in enumerate(model.layers):
            lp = f"{pre}.layers.{i}"
            put(layer.input_norm.weight, index.get(f"{lp}.input_layernorm.weight"))
            put(layer.post_norm.weight, index.get(f"{lp}.post_attention_layernorm.weight"))
            used += _load_mlp(index, layer.mlp, f"{lp}.mlp", put)
            a = layer.attn
            if isinstance(a, GatedDeltaNet):
                la = f"{lp}.linear_attn"
                kd, vd = a.key_dim * tp, a.value_dim * tp        # full widths in the checkpoint
                q, k, v = index.get(f"{la}.in_proj_qkv.weight").split([kd, kd, vd], 0)
                put(a.in_qkvz, torch.cat([_sh0(q), _sh0(k), _sh0(v), _sh0(index.get(f"{la}.in_proj_z.weight"))], 0))
                put(a.in_ba, torch.cat([_sh0(index.get(f"{la}.in_proj_b.weight")), _sh0(index.get(f"{la}.in_proj_a.weight"))], 0))
                cq, ck, cv = index.get(f"{la}.conv1d.weight").reshape(2 * kd + vd, a.k).split([kd, kd, vd], 0)
                put(a.conv_weight, torch.cat([_sh0(cq), _sh0(ck), _sh0(cv)], 0))
                put(a.dt_bias, _sh0(index.get(f"{la}.dt_bias")))
                put(a.A_log, _sh0(index.get(f"{la}.A_log")))
                put(a.norm_weight, index.get(f"{la}.norm.weight"))
                put(a.out_proj.weight, _sh1(index.get(f"{la}.out_proj.weight")))
            else:
                sa = f"{lp}.self_attn"
                qw = index.get(f"{sa}.q_proj.weight")
                d, hq, hkv, rep = a.d, a.hq, a.hkv, a.qkv.kv_rep     # local head counts
                if a.gate is not None:
                    qg = qw.view(hq * tp, 2, d, qw.shape[-1])[rank * hq:(rank + 1) * hq]
                    qw = qg[:, 0].reshape(hq * d, -1)
                    put(a.gate.weight, qg[:, 1].reshape(hq * d, -1))
                else:
                    qw = _sh0(qw)
                kv_lo = (rank // rep) * hkv * d
                kw = index.get(f"{sa}.k_proj.weight")[kv_lo:kv_lo + hkv * d]
                vw = index.get(f"{sa}.v_proj.weight")[kv_lo:kv_lo + hkv * d]
                put(a.qkv.weight, torch.cat([qw, kw, vw], 0))
                put(a.o.weight, _sh1(index.get(f"{sa}.o_proj.weight")))
                put(a.q_norm.weight, index.get(f"{sa}.q_norm.weight"))
                put(a.k_norm.weight, index.get(f"{sa}.k_norm.weight"))
            if i % 8 == 7:
                index.drop()
        index.drop()
        logger.info("checkpoint loaded path=%s tensors=%d prefix=%s", path, used, pre)

    # ------------------------------------------------------------------ save
    @torch.no_grad()
    def save_weights(self, model, path, config, source_path=None):
        from safetensors.torch import save_file

        from ..engine.checkpoint import _passthrough_untouched, copy_assets
        from ..parallel.context import get_context

        ctx = get_context()
        import torch.distributed as dist

        if ctx.dp_rank != 0:
            if ctx.world_size > 1:
                dist.barrier()
            return
        writer = ctx.tp_rank == 0          # every rank of the group takes part in the gathers, one writes
        tp = ctx.tp_size
        os.makedirs(path, exist_ok=True)
        pre = config.checkpoint_prefix or "model"
        out: dict[str, torch.Tensor] = {}

        def cpu(t):
            return t.detach().to("cpu", copy=True).contiguous() if writer else t

        vocab = config.vocab_size
        out[f"{pre}.embed_tokens.weight"] = cpu(_full(model.embed.weight, 0)[:vocab])
        out[f"{pre}.norm.weight"] = cpu(model.norm.weight)
        if not config.tie_word_embeddings:
            out["lm_head.weight"] = cpu(_full(model.lm_head.weight, 0)[:vocab])
        for i, layer in enumerate(model.layers):
            lp = f"{pre}.layers.{i}"
            out[f"{lp}.input_layernorm.weight"] = cpu(layer.input_norm.weight)
            out[f"{lp}.post_attention_layernorm.weight"] = cpu(layer.post_norm.weight)
            _save_mlp(out, layer.mlp, f"{lp}.mlp", cpu)
            a = layer.attn
            if isinstance(a, GatedDeltaNet):
                la = f"{lp}.linear_attn"
                kd, vd = a.key_dim, a.value_dim       # local widths
                q, k, v, z = a.in_qkvz.split([kd, kd, vd, vd], 0)
                out[f"{la}.in_proj_qkv.weight"] = cpu(torch.cat([_full(q), _full(k), _full(v)], 0))
                out[f"{la}.in_proj_z.weight"] = cpu(_full(z))
                out[f"{la}.in_proj_b.weight"] = cpu(_full(a.in_ba[: a.hv]))
                out[f"{la}.in_proj_a.weight"] = cpu(_full(a.in_ba[a.hv:]))
                cq, ck, cv = a.conv_weight.split([kd, kd, vd], 0)
                out[f"{la}.conv1d.weight"] = cpu(torch.cat([_full(cq), _full(ck), _full(cv)], 0).reshape(-1, 1, a.k))
                out[f"{la}.dt_bias"] = cpu(_full(a.dt_bias))
                out[f"{la}.A_log"] = cpu(_full(a.A_log))
                out[f"{la}.norm.weight"] = cpu(a.norm_weight)
                out[f"{la}.out_proj.weight"] = cpu(_full(a.out_proj.weight, 1))
            else:
                sa = f"{lp}.self_attn"
                d, hq, hkv, rep = a.d, a.hq, a.hkv, a.qkv.kv_rep
                qw = a.qkv.weight[: hq * d]
                if a.gate is not None:
                    qw = torch.stack([qw.view(hq, d, -1), a.gate.weight.view(hq, d, -1)], 1).reshape(2 * hq * d, -1)
                out[f"{sa}.q_proj.weight"] = cpu(_full(qw))
                out[f"{sa}.k_proj.weight"] = cpu(_full_kv(a.qkv.weight[hq * d:(hq + hkv) * d], rep))
                out[f"{sa}.v_proj.weight"] = cpu(_full_kv(a.qkv.weight[(hq + hkv) * d:], rep))
                out[f"{sa}.o_proj.weight"] = cpu(_full(a.o.weight, 1))
                out[f"{sa}.q_norm.weight"] = cpu(a.q_norm.weight)
                out[f"{sa}.k_norm.weight"] = cpu(a.k_norm.weight)
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

    def hf_config(self, config: ModelConfig) -> dict[str, Any]:
        return _hf_text_config(config)


class Qwen35Adapter(_HybridAdapter):
    name = "qwen3_5"

    def match_hf_config(self, hf):
        return str(hf.get("model_type", "")).lower() == "qwen3_5" or \
            "Qwen3_5ForConditionalGeneration" in set(hf.get("architectures") or [])

    def config_from_hf(self, hf):
        return _text_config(hf, self.name, "model")


class MiniCPMV46Adapter(_HybridAdapter):
    """Text trunk of the MiniCPM-V 4.6 vision-language model; vision tensors pass through on save."""

    name = "minicpmv46"
    prefixes = ("model.language_model", "model")

    def match_hf_config(self, hf):
        return str(hf.get("model_type", "")).lower() == "minicpmv4_6"

    def config_from_hf(self, hf):
        return _text_config(hf, self.name, "model.language_model")

    def hf_config(self, config):
        return {"model_type": "minicpmv4_6", "text_config": _hf_text_config(config)}


class Qwen35MoeAdapter(_HybridAdapter):
    """Qwen3.5-MoE: the hybrid stack with a sparse block in every layer (softmax top-k router, routed
    experts, shared expert scaled by a per-token sigmoid gate); reference
    ``areno/models/qwen3_5/model.py:499-547,883-940``."""

    name = "qwen3_5_moe"

    def match_hf_config(self, hf):
        return str(hf.get("model_type", "")).lower() == "qwen3_5_moe" or \
            "Qwen3_5MoeForConditionalGeneration" in set(hf.get("architectures") or [])

    def config_from_hf(self, hf):
        text = hf.get("text_config") or hf
        hf2 = dict(hf)
        t2 = dict(text)
        t2.setdefault("intermediate_size", text.get("shared_expert_intermediate_size", text["moe_intermediate_size"]))
        if "text_config" in hf:
            hf2["text_config"] = t2
        else:
            hf2 = t2
        cfg = _text_config(hf2, self.name, "model")
        cfg.num_experts = int(text["num_experts"])
        cfg.num_experts_per_tok = int(text.get("num_experts_per_tok", 8))
        cfg.moe_intermediate_size = int(text["moe_intermediate_size"])
        cfg.shared_expert_intermediate_size = int(text.get("shared_expert_intermediate_size", 0) or 0)
        cfg.norm_topk_prob = bool(text.get("norm_topk_prob", True))
        cfg.extra = dict(cfg.extra or {}, shared_expert_gate=cfg.shared_expert_intermediate_size > 0)
        return cfg


ADAPTERS = [Qwen35MoeAdapter, Qwen35Adapter, MiniCPMV46Adapter]
