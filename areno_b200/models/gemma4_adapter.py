"""Adapter for Gemma-4 text checkpoints (``model_type`` ``gemma4`` / ``gemma4_unified`` / ``gemma4_text``;
reference: ``areno/models/gemma4/model.py:820-905`` and ``checkpoint.py``).  Multimodal checkpoints keep
the text trunk under ``model.language_model``; vision / audio tensors pass through untouched on save.
Loads and saves at tensor-parallel size 1."""

from __future__ import annotations

import json
import os
from typing import Any

import torch

from ..engine.config import ModelConfig, parse_dtype
from .base import ModelAdapter
from .gemma4 import Gemma4CausalLM

_LAYER_NORMS = (("input_norm", "input_layernorm"), ("post_attn_norm", "post_attention_layernorm"),
                ("pre_ff_norm", "pre_feedforward_layernorm"), ("post_ff_norm", "post_feedforward_layernorm"),
                ("pre_ff_norm_2", "pre_feedforward_layernorm_2"), ("post_ff_norm_1", "post_feedforward_layernorm_1"),
                ("post_ff_norm_2", "post_feedforward_layernorm_2"), ("post_ple_norm", "post_per_layer_input_norm"))


def _tensor_plan(model: Gemma4CausalLM, cfg: ModelConfig, pre: str):
    """Yield ``(hf_key, getter, setter, kind)`` describing every tensor of the text trunk.  ``getter`` / ``setter``
    address this rank's part; ``kind`` says how that part sits in the full tensor: ``rep`` (replicated), ``rows`` /
    ``cols`` (equal shares of dim 0 / dim 1 in rank order; experts are rows), ``vocab:<n>`` (row shares of a table
    padded beyond its ``n`` valid rows) and ``kv:<rep>`` (row shares that ``rep`` neighbouring ranks hold copies of).
    ``_local_part`` / ``_full_tensor`` also know ``parts:<n>`` (``n`` equal row blocks, each shared out by rows) and
    ``qkv:<q>:<kv>:<rep>`` (a fused q | k | v tensor: ``q`` local query rows, ``kv`` local key rows, replication).
    """
    vocab = cfg.vocab_size

    def whole(param):
        return (lambda: param.detach()), (lambda t: param.copy_(t.to(param.dtype)))

    def rows(param, lo, hi):
        return (lambda: param.detach()[lo:hi]), (lambda t: param[lo:hi].copy_(t.to(param.dtype)))

    yield (f"{pre}.embed_tokens.weight", *whole(model.embed.weight), f"vocab:{vocab}")
    yield (f"{pre}.norm.weight", *whole(model.norm.weight), "rep")
    if not cfg.tie_word_embeddings:
        yield ("lm_head.weight", *whole(model.lm_head.weight), f"vocab:{vocab}")
    if model.ple > 0:
        yield (f"{pre}.embed_tokens_per_layer.weight", *whole(model.embed_per_layer.weight), f"vocab:{model.ple_vocab}")
        yield (f"{pre}.per_layer_model_projection.weight", *whole(model.per_layer_model_projection.weight), "rep")
        yield (f"{pre}.per_layer_projection_norm.weight", *whole(model.per_layer_projection_norm.weight), "rep")
    for i, layer in enumerate(model.layers):
        lp = f"{pre}.layers.{i}"
        for attr, name in _LAYER_NORMS:
            mod = getattr(layer, attr)
            if mod is not None:
                yield (f"{lp}.{name}.weight", *whole(mod.weight), "rep")
        a = layer.attn
        q, kv = a.hq * a.d, a.hkv * a.d
        yield (f"{lp}.self_attn.q_proj.weight", *rows(a.qkv.weight, 0, q), "rows")
        yield (f"{lp}.self_attn.k_proj.weight", *rows(a.qkv.weight, q, q + kv), f"kv:{a.qkv.kv_rep}")
        yield (f"{lp}.self_attn.v_proj.weight", *rows(a.qkv.weight, q + kv, q + 2 * kv), f"kv:{a.qkv.kv_rep}")
        yield (f"{lp}.self_attn.o_proj.weight", *whole(a.o.weight), "cols")
        yield (f"{lp}.self_attn.q_norm.weight", *whole(a.q_norm.weight), "rep")
        yield (f"{lp}.self_attn.k_norm.weight", *whole(a.k_norm.weight), "rep")
        inter = layer.mlp.gate_up.weight.shape[0] // 2
        yield (f"{lp}.mlp.gate_proj.weight", *rows(layer.mlp.gate_up.weight, 0, inter), "rows")
        yield (f"{lp}.mlp.up_proj.weight", *rows(layer.mlp.gate_up.weight, inter, 2 * inter), "rows")
        yield (f"{lp}.mlp.down_proj.weight", *whole(layer.mlp.down.weight), "cols")
        if layer.ple_gate is not None:
            yield (f"{lp}.per_layer_input_gate.weight", *whole(layer.ple_gate.weight), "rep")
            yield (f"{lp}.per_layer_projection.weight", *whole(layer.ple_proj.weight), "rep")
        yield (f"{lp}.layer_scalar", *whole(layer.layer_scalar), "rep")
        if layer.moe is not None:
            yield (f"{lp}.router.scale", *whole(layer.router.scale), "rep")
            yield (f"{lp}.router.proj.weight", *whole(layer.router.proj.weight), "rep")
            yield (f"{lp}.router.per_expert_scale", *whole(layer.moe.per_expert_scale), "rep")
            yield (f"{lp}.experts.gate_up_proj", *whole(layer.moe.gate_up), "rows")
            yield (f"{lp}.experts.down_proj", *whole(layer.moe.down), "rows")


def _local_part(full: torch.Tensor, local_shape, kind: str, tp: int, rank: int) -> torch.Tensor:
    """This rank's part of a checkpoint tensor, shaped like the local parameter (slice)."""
    if tp == 1 and not kind.startswith("vocab"):
        return full.reshape(local_shape)
    if kind == "rep":
        return full.reshape(local_shape)
    if kind == "rows":
        return full.chunk(tp, 0)[rank].reshape(local_shape)
    if kind == "cols":
        return full.chunk(tp, 1)[rank].reshape(local_shape)
    if kind.startswith("kv:"):
        rep = int(kind[3:])
        n = local_shape[0]
        lo = (rank // rep) * n
        return full[lo:lo + n].reshape(local_shape)
    if kind.startswith("parts:"):
        n = int(kind[6:])
        return torch.cat([part.chunk(tp, 0)[rank] for part in full.chunk(n, 0)], 0).reshape(local_shape)
    if kind.startswith("qkv:"):
        q, kv, rep = (int(v) for v in kind[4:].split(":"))
        q_full, kv_full = q * tp, kv * (tp // rep)
        k_lo = q_full + (rank // rep) * kv
        v_lo = q_full + kv_full + (rank // rep) * kv
        return torch.cat([full[rank * q:(rank + 1) * q], full[k_lo:k_lo + kv], full[v_lo:v_lo + kv]], 0).reshape(local_shape)
    if kind.startswith("vocab:"):
        valid, per = int(kind[6:]), local_shape[0]
        out = torch.zeros(local_shape, dtype=full.dtype)
        lo, hi = min(rank * per, valid), min((rank + 1) * per, valid)
        if hi > lo:
            out[: hi - lo] = full[lo:hi]
        return out
    raise ValueError(f"unknown kind {kind}")


def _full_tensor(local: torch.Tensor, kind: str) -> torch.Tensor:
    """The checkpoint tensor rebuilt from the ranks' parts (a collective inside the TP group)."""
    from .hybrid_adapters import _full, _full_kv

    if kind == "rep":
        return local
    if kind == "rows":
        return _full(local, 0)
    if kind == "cols":
        return _full(local, 1)
    if kind.startswith("kv:"):
        return _full_kv(local, int(kind[3:]))
    if kind.startswith("parts:"):
        return torch.cat([_full(part, 0) for part in local.chunk(int(kind[6:]), 0)], 0)
    if kind.startswith("qkv:"):
        q, kv, rep = (int(v) for v in kind[4:].split(":"))
        return torch.cat([_full(local[:q], 0), _full_kv(local[q:q + kv], rep), _full_kv(local[q + kv:], rep)], 0)
    if kind.startswith("vocab:"):
        return _full(local, 0)[: int(kind[6:])]
    raise ValueError(f"unknown kind {kind}")


# keys that older / alternative exports use for the same tensor
_ALIASES = {"router.scale": ("router.scale.weight",), "router.proj.weight": ("router.weight",),
            "router.per_expert_scale": ("moe.per_expert_scale",), "experts.gate_up_proj": ("experts.gate_up_proj.weight",),
            "experts.down_proj": ("experts.down_proj.weight",)}
_OPTIONAL = ("layer_scalar",)


class Gemma4Adapter(ModelAdapter):
    name = "gemma4"

    def match_hf_config(self, hf):
        types = {str(hf.get("model_type", "")).lower(), str((hf.get("text_config") or {}).get("model_type", "")).lower()}
        return bool(types & {"gemma4", "gemma4_unified", "gemma4_text"})

    def config_from_hf(self, hf) -> ModelConfig:
        text = hf.get("text_config")
        prefix = "model.language_model" if isinstance(text, dict) else "model"
        c = text if isinstance(text, dict) else hf
        act = str(c.get("hidden_activation", c.get("hidden_act", "gelu_pytorch_tanh")))
        if act != "gelu_pytorch_tanh":
            raise ValueError("Gemma-4 support requires hidden_activation='gelu_pytorch_tanh'")
        if c.get("swa_head_dim") is not None and c.get("global_head_dim") is not None:
            raise ValueError("use either global_head_dim or swa_head_dim, not both")
        heads = int(c["num_attention_heads"])
        n = int(c["num_hidden_layers"])
        base_d = int(c.get("head_dim", int(c["hidden_size"]) // heads))
        moe = bool(c.get("enable_moe_block", False))
        topk = c.get("top_k_experts", c.get("num_experts_per_tok"))
        return ModelConfig(
            model_type=self.name, checkpoint_prefix=prefix, vocab_size=int(c["vocab_size"]), hidden_size=int(c["hidden_size"]),
            intermediate_size=int(c["intermediate_size"]), num_hidden_layers=n, num_attention_heads=heads,
            num_key_value_heads=int(c.get("num_global_key_value_heads") or c.get("num_key_value_heads", heads)),
            head_dim=int(c.get("global_head_dim") or base_d), rms_norm_eps=float(c.get("rms_norm_eps", 1e-6)),
            rope_theta=float(c.get("rope_theta", 10000.0)), max_position_embeddings=int(c.get("max_position_embeddings", 131072)),
            tie_word_embeddings=bool(c.get("tie_word_embeddings", True)), qkv_bias=bool(c.get("attention_bias", False)),
            qk_norm=True, v_norm=True,
            dtype=parse_dtype(hf.get("torch_dtype") or c.get("torch_dtype") or hf.get("dtype") or c.get("dtype")),
            hidden_act="gelu_tanh", layer_types=tuple(c.get("layer_types") or ("full_attention",) * n),
            sliding_window=c.get("sliding_window"), swa_head_dim=int(c.get("swa_head_dim") or base_d),
            swa_num_key_value_heads=int(c.get("swa_num_key_value_heads") or c.get("num_key_value_heads", heads)),
            rope_parameters=c.get("rope_parameters"), attention_k_eq_v=bool(c.get("attention_k_eq_v", False)),
            num_kv_shared_layers=int(c.get("num_kv_shared_layers") or 0),
            partial_rotary_factor=float(c.get("partial_rotary_factor", 1.0)),
            hidden_size_per_layer_input=int(c.get("hidden_size_per_layer_input") or 0),
            vocab_size_per_layer_input=c.get("vocab_size_per_layer_input"),
            use_double_wide_mlp=bool(c.get("use_double_wide_mlp", False)), enable_moe_block=moe,
            num_experts=int(c["num_experts"]) if moe and c.get("num_experts") is not None else None,
            num_experts_per_tok=int(topk) if moe and topk is not None else 1,
            moe_intermediate_size=int(c.get("moe_intermediate_size") or 0) if moe else 0,
            norm_topk_prob=bool(c.get("norm_topk_prob", True)), attention_softmax_scale=1.0,
            final_logit_softcapping=c.get("final_logit_softcapping"))

    def build(self, config, device="cpu"):
        if config.enable_moe_block and not (config.num_experts and config.moe_intermediate_size > 0):
            raise ValueError("Gemma-4 MoE requires num_experts and moe_intermediate_size")
        return Gemma4CausalLM(config, device=device)

    @staticmethod
    def _find(index, pre: str, key: str, cfg: ModelConfig):
        if key in index:
            return key
        tail = key.split(".layers.", 1)[-1].split(".", 1)[-1] if ".layers." in key else key
        for alt in _ALIASES.get(tail, ()):
            cand = key[: len(key) - len(tail)] + alt
            if cand in index:
                return cand
        if key == "lm_head.weight" and f"{pre}.lm_head.weight" in index:
            return f"{pre}.lm_head.weight"
        if key.endswith("self_attn.v_proj.weight") and cfg.attention_k_eq_v:
            return key.replace("v_proj", "k_proj")
        return None

    @torch.no_grad()
    def load_weights(self, model, path, config):
        from ..engine.checkpoint import SafetensorsIndex, logger
        from ..parallel.context import get_context

        ctx = get_context()
        index = SafetensorsIndex(path)
        pre = next(p for p in (config.checkpoint_prefix, "model", "model.language_model") if f"{p}.embed_tokens.weight" in index)
        used = 0
        for n_seen, (key, _get, put, kind) in enumerate(_tensor_plan(model, config, pre)):
            found = self._find(index, pre, key, config)
            if found is None:
                if key.rsplit(".", 1)[-1] in _OPTIONAL or key.endswith(_OPTIONAL):
                    continue
                raise KeyError(f"checkpoint is missing {key}")
            put(_local_part(index.get(found), tuple(_get().shape), kind, ctx.tp_size, ctx.tp_rank))
            used += 1
            if n_seen % 256 == 255:
                index.drop()
        index.drop()
        logger.info("checkpoint loaded path=%s tensors=%d prefix=%s", path, used, pre)

    @torch.no_grad()
    def save_weights(self, model, path, config, source_path=None):
        from safetensors.torch import save_file

        from ..engine.checkpoint import _passthrough_untouched, copy_assets
        from ..parallel.context import get_context

        import torch.distributed as dist

        ctx = get_context()
        if ctx.dp_rank != 0:
            if ctx.world_size > 1:
                dist.barrier()
            return
        os.makedirs(path, exist_ok=True)
        pre = config.checkpoint_prefix or "model"
        writer = ctx.tp_rank == 0        # every rank of the TP group takes part in the gathers, one writes
        out = {}
        for key, get, _put, kind in _tensor_plan(model, config, pre):
            full = _full_tensor(get(), kind)
            if writer:
                out[key] = full.to("cpu", copy=True).contiguous()
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
        text = {
            "model_type": "gemma4_text", "vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
            "intermediate_size": c.intermediate_size, "num_hidden_layers": c.num_hidden_layers,
            "num_attention_heads": c.num_attention_heads, "num_key_value_heads": c.swa_num_key_value_heads or c.num_key_value_heads,
            "num_global_key_value_heads": c.num_key_value_heads, "head_dim": c.swa_head_dim or c.head_dim,
            "global_head_dim": c.head_dim, "rms_norm_eps": c.rms_norm_eps, "rope_theta": c.rope_theta,
            "max_position_embeddings": c.max_position_embeddings, "tie_word_embeddings": c.tie_word_embeddings,
            "attention_bias": c.qkv_bias, "hidden_activation": "gelu_pytorch_tanh", "layer_types": list(c.layer_types or []),
            "sliding_window": c.sliding_window, "rope_parameters": c.rope_parameters, "attention_k_eq_v": c.attention_k_eq_v,
            "num_kv_shared_layers": c.num_kv_shared_layers, "partial_rotary_factor": c.partial_rotary_factor,
            "hidden_size_per_layer_input": c.hidden_size_per_layer_input, "vocab_size_per_layer_input": c.vocab_size_per_layer_input,
            "use_double_wide_mlp": c.use_double_wide_mlp, "enable_moe_block": c.enable_moe_block, "num_experts": c.num_experts,
            "top_k_experts": c.num_experts_per_tok, "moe_intermediate_size": c.moe_intermediate_size,
            "norm_topk_prob": c.norm_topk_prob, "final_logit_softcapping": c.final_logit_softcapping,
            "torch_dtype": str(c.dtype).replace("torch.", ""),
        }
        if (c.checkpoint_prefix or "model") == "model":
            return dict(text, model_type="gemma4")
        return {"model_type": "gemma4", "text_config": text}


ADAPTERS = [Gemma4Adapter]
