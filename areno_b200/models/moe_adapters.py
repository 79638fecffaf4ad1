"""Adapter for Qwen3-MoE checkpoints (``model_type == "qwen3_moe"``; reference:
``areno/models/qwen3/model.py:443-491`` and ``checkpoint.py``).  HF stores one tensor per expert and
projection; here they are stacked into ``[experts_local, 2 * inter, hidden]`` (gate over up) and
``[experts_local, hidden, inter]`` so that one grouped GEMM serves all local experts."""

from __future__ import annotations

import torch

from .dense_adapters import _DenseAdapter, _common
from .moe import MoeCausalLM, SparseMoeBlock

_EXPERT = "model.layers.{layer}.mlp.experts.{expert}.{proj}.weight"
_GATE = "model.layers.{layer}.mlp.gate.weight"


def _load_layer_experts(index, layer, i: int) -> int:
    mlp = layer.mlp
    if not isinstance(mlp, SparseMoeBlock):
        return 0
    used = 0
    with torch.no_grad():
        mlp.router.weight.copy_(index.get(_GATE.format(layer=i)).to(torch.float32))
        used += 1
        ex = mlp.experts
        inter = ex.inter
        for le in range(ex.e_local):
            e = ex.e_lo + le
            ex.gate_up[le, :inter].copy_(index.get(_EXPERT.format(layer=i, expert=e, proj="gate_proj")))
            ex.gate_up[le, inter:].copy_(index.get(_EXPERT.format(layer=i, expert=e, proj="up_proj")))
            ex.down[le].copy_(index.get(_EXPERT.format(layer=i, expert=e, proj="down_proj")))
            used += 3
    return used


def _export_layer_experts(layer, i: int) -> dict[str, torch.Tensor]:
    from ..parallel.context import get_context

    mlp = layer.mlp
    if not isinstance(mlp, SparseMoeBlock):
        return {}
    out: dict[str, torch.Tensor] = {}
    ctx = get_context()
    if ctx.tp_rank == 0 and (ctx.ep_size == 1 or ctx.ep_rank == 0):      # the router is replicated: one writer
        out[_GATE.format(layer=i)] = mlp.router.weight.detach().to("cpu", copy=True)
    ex = mlp.experts
    inter = ex.inter
    for le in range(ex.e_local):
        e = ex.e_lo + le
        gu = ex.gate_up[le].detach()
        out[_EXPERT.format(layer=i, expert=e, proj="gate_proj")] = gu[:inter].to("cpu", copy=True).contiguous()
        out[_EXPERT.format(layer=i, expert=e, proj="up_proj")] = gu[inter:].to("cpu", copy=True).contiguous()
        out[_EXPERT.format(layer=i, expert=e, proj="down_proj")] = ex.down[le].detach().to("cpu", copy=True).contiguous()
    return out


class Qwen3MoeAdapter(_DenseAdapter):
    name = "qwen3_moe"
    model_types = ("qwen3_moe",)

    def config_from_hf(self, hf):
        return _common(
            hf, model_type="qwen3_moe", qk_norm=bool(hf.get("qk_layernorm", True)),
            qkv_bias=bool(hf.get("attention_bias", False)), rope_theta=float(hf.get("rope_theta", 1_000_000.0)),
            num_experts=int(hf["num_experts"]), num_experts_per_tok=int(hf.get("num_experts_per_tok", 8)),
            moe_intermediate_size=int(hf["moe_intermediate_size"]), norm_topk_prob=bool(hf.get("norm_topk_prob", True)),
            extra={"decoder_sparse_step": int(hf.get("decoder_sparse_step", 1) or 1),
                   "mlp_only_layers": list(hf.get("mlp_only_layers") or [])})

    def build(self, config, device="cpu"):
        return MoeCausalLM(config, device=device)

    def load_weights(self, model, path, config):
        from ..engine.checkpoint import DENSE_LAYER, DENSE_TOP, Rule, load_with_rules, logger

        top = list(DENSE_TOP)
        if not config.tie_word_embeddings:
            top.append(Rule("lm_head.weight", (config.checkpoint_lm_head_key,), "vocab"))
        n = load_with_rules(model, path, top, DENSE_LAYER, config.num_hidden_layers, expert_rules=_load_layer_experts)
        logger.info("checkpoint loaded path=%s tensors=%d", path, n)

    def save_weights(self, model, path, config, source_path=None):
        from ..engine.checkpoint import DENSE_LAYER, DENSE_TOP, Rule, save_with_rules

        top = list(DENSE_TOP)
        if not config.tie_word_embeddings:
            top.append(Rule("lm_head.weight", (config.checkpoint_lm_head_key,), "vocab"))
        save_with_rules(model, path, config, top, DENSE_LAYER, config.num_hidden_layers, source_path,
                        expert_export=_export_layer_experts)


ADAPTERS = [Qwen3MoeAdapter]
