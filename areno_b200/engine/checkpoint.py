"""Hugging Face safetensors checkpoints: sliced load into TP shards, distributed save.

A model family describes its tensors with ``Rule`` objects (HF key pattern -> module attribute,
plus how the local tensor maps onto the full one).  Loading reads only this rank's slice of each
tensor (``safe_open(...).get_slice``); fused projections (QKV, gate_up) are assembled from their HF
parts.  Saving gathers shards over the TP group to a per-tensor owner (``crc32(key) % tp``), each TP
rank of DP row 0 writes ``model-{rank+1:05d}-of-{tp:05d}.safetensors``, and rank 0 writes the merged
``model.safetensors.index.json`` carrying ``areno_checkpoint_writer: distributed_tp`` and copies the
tokenizer / config assets - the on-disk contract of the reference
(``areno/engine/checkpoints/io.py:582-670``, ``common.py:48-205``).
"""

from __future__ import annotations

import json
import os
import shutil
import zlib
from dataclasses import dataclass
from typing import Any, Callable

import torch
import torch.distributed as dist

from ..parallel.context import get_context
from ..utils.log import get_logger

logger = get_logger()

ASSET_FILES = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "vocab.json",
               "merges.txt", "special_tokens_map.json", "added_tokens.json", "tokenizer.model", "chat_template.jinja",
               "chat_template.json", "preprocessor_config.json", "processor_config.json")


# ------------------------------------------------------------------------ reading
class SafetensorsIndex:
    """Lazy key -> file map over a single-file or sharded safetensors checkpoint."""

    def __init__(self, path: str):
        from safetensors import safe_open

        self.path = path
        self._open = safe_open
        self._handles: dict[str, Any] = {}
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self.weight_map: dict[str, str] = json.load(f)["weight_map"]
        else:
            self.weight_map = {}
            for fname in sorted(os.listdir(path)):
                if fname.endswith(".safetensors"):
                    with safe_open(os.path.join(path, fname), framework="pt") as f:
                        for k in f.keys():
                            self.weight_map[k] = fname
        if not self.weight_map:
            raise FileNotFoundError(f"no safetensors weights under {path}")

    def __contains__(self, key: str) -> bool:
        return key in self.weight_map

    def keys(self):
        return self.weight_map.keys()

    def _handle(self, key: str):
        fname = self.weight_map[key]
        h = self._handles.get(fname)
        if h is None:
            h = self._open(os.path.join(self.path, fname), framework="pt")
            self._handles[fname] = h
        return h

    def get(self, key: str) -> torch.Tensor:
        return self._handle(key).get_tensor(key)

    def get_rows(self, key: str, lo: int, hi: int) -> torch.Tensor:
        return self._handle(key).get_slice(key)[lo:hi]

    def get_cols(self, key: str, lo: int, hi: int) -> torch.Tensor:
        return self._handle(key).get_slice(key)[:, lo:hi]

    def shape(self, key: str) -> list[int]:
        return list(self._handle(key).get_slice(key).get_shape())

    def drop(self) -> None:
        self._handles.clear()


# -------------------------------------------------------------------------- rules
@dataclass
class Rule:
    """How one local parameter maps onto HF tensors.

    kind: ``replicated`` | ``rows`` (dim-0 shard) | ``cols`` (dim-1 shard) | ``vocab`` (dim-0 shard, zero
    padded) | ``merged_rows`` (several HF tensors, each dim-0 sharded, concatenated) | ``qkv`` (q heads
    sharded, k / v heads sharded or replicated).  ``keys`` may contain ``{layer}`` / ``{expert}``.
    """

    attr: str
    keys: tuple[str, ...]
    kind: str = "replicated"
    optional: bool = False


def _resolve(module, attr: str):
    obj = module
    for part in attr.split("."):
        obj = obj[int(part)] if part.isdigit() else getattr(obj, part)
    return obj


def _shard_bounds(total: int, tp: int, rank: int) -> tuple[int, int]:
    if total % tp != 0:
        raise ValueError(f"a dimension of {total} cannot be split evenly over tp={tp}")
    per = total // tp
    return rank * per, (rank + 1) * per


def load_rule(index: SafetensorsIndex, param: torch.Tensor, rule: Rule, keys: tuple[str, ...], qkv_meta=None) -> bool:
    ctx = get_context()
    tp, r = ctx.tp_size, ctx.tp_rank
    if any(k not in index for k in keys):
        if rule.optional:
            return False
        missing = [k for k in keys if k not in index]
        raise KeyError(f"checkpoint is missing {missing}")
    if rule.kind == "replicated":
        t = index.get(keys[0])
    elif rule.kind == "rows":
        lo, hi = _shard_bounds(index.shape(keys[0])[0], tp, r)
        t = index.get_rows(keys[0], lo, hi)
    elif rule.kind == "cols":
        lo, hi = _shard_bounds(index.shape(keys[0])[1], tp, r)
        t = index.get_cols(keys[0], lo, hi)
    elif rule.kind == "vocab":
        total = index.shape(keys[0])[0]
        per = param.shape[0]
        lo, hi = min(r * per, total), min((r + 1) * per, total)
        t = torch.zeros(param.shape, dtype=param.dtype)
        if hi > lo:
            t[: hi - lo] = index.get_rows(keys[0], lo, hi)
    elif rule.kind == "merged_rows":
        parts = []
        for k in keys:
            lo, hi = _shard_bounds(index.shape(k)[0], tp, r)
            parts.append(index.get_rows(k, lo, hi))
        t = torch.cat(parts, dim=0)
    elif rule.kind == "qkv":
        if len(qkv_meta) > 4:
            raise ValueError("an uneven (padded) head layout is inference-only and is filled from a full replica")
        hq_rows, hkv, d, rep = qkv_meta          # local q rows (heads * q_mult), local kv heads, head_dim, kv replication
        q_rows = hq_rows * d
        q = index.get_rows(keys[0], r * q_rows, (r + 1) * q_rows)
        kv_rank = r // rep
        k = index.get_rows(keys[1], kv_rank * hkv * d, (kv_rank + 1) * hkv * d)
        v = index.get_rows(keys[2], kv_rank * hkv * d, (kv_rank + 1) * hkv * d)
        t = torch.cat([q, k, v], dim=0)
    else:
        raise ValueError(f"unknown rule kind {rule.kind}")
    if tuple(t.shape) != tuple(param.shape):
        raise ValueError(f"shape mismatch for {keys}: checkpoint slice {tuple(t.shape)} vs parameter {tuple(param.shape)}")
    with torch.no_grad():
        param.copy_(t.to(param.dtype))
    return True


def load_with_rules(model, path: str, top_rules: list[Rule], layer_rules: list[Rule], num_layers: int,
                    layers_attr: str = "layers", expert_rules: Callable | None = None) -> int:
    """Apply rules; returns the number of HF tensors consumed."""
    index = SafetensorsIndex(path)
    used = 0

    def apply(rule: Rule, prefix_obj, fmt: dict):
        nonlocal used
        try:
            param = _resolve(prefix_obj, rule.attr)
        except AttributeError:
            if rule.optional:
                return
            raise
        if param is None:
            return
        keys = tuple(k.format(**fmt) for k in rule.keys)
        meta = None
        if rule.kind == "qkv":
            shard = getattr(param, "tp_shard", None)
            meta = shard[1] if shard else None
        if load_rule(index, param, rule, keys, meta):
            used += len(keys)

    for rule in top_rules:
        apply(rule, model, {})
    layers = _resolve(model, layers_attr)
    for i in range(num_layers):
        for rule in layer_rules:
            apply(rule, layers[i], {"layer": i})
        if expert_rules is not None:
            used += expert_rules(index, layers[i], i)
        if i % 8 == 7:
            index.drop()   # bound the number of open mmaps / cached handles
    index.drop()
    return used


# ------------------------------------------------------------------------- dense
DENSE_TOP = [
    Rule("embed.weight", ("model.embed_tokens.weight",), "vocab"),
    Rule("norm.weight", ("model.norm.weight",), "replicated"),
]
DENSE_LAYER = [
    Rule("input_norm.weight", ("model.layers.{layer}.input_layernorm.weight",)),
    Rule("post_norm.weight", ("model.layers.{layer}.post_attention_layernorm.weight",)),
    Rule("attn.qkv.weight", ("model.layers.{layer}.self_attn.q_proj.weight", "model.layers.{layer}.self_attn.k_proj.weight",
                             "model.layers.{layer}.self_attn.v_proj.weight"), "qkv"),
    Rule("attn.qkv.bias", ("model.layers.{layer}.self_attn.q_proj.bias", "model.layers.{layer}.self_attn.k_proj.bias",
                           "model.layers.{layer}.self_attn.v_proj.bias"), "qkv", optional=True),
    Rule("attn.q_norm.weight", ("model.layers.{layer}.self_attn.q_norm.weight",), optional=True),
    Rule("attn.k_norm.weight", ("model.layers.{layer}.self_attn.k_norm.weight",), optional=True),
    Rule("attn.o.weight", ("model.layers.{layer}.self_attn.o_proj.weight",), "cols"),
    Rule("mlp.gate_up.weight", ("model.layers.{layer}.mlp.gate_proj.weight", "model.layers.{layer}.mlp.up_proj.weight"),
         "merged_rows", optional=True),
    Rule("mlp.down.weight", ("model.layers.{layer}.mlp.down_proj.weight",), "cols", optional=True),
]


def load_dense_checkpoint(model, path: str, config) -> None:
    top = list(DENSE_TOP)
    if not config.tie_word_embeddings:
        top.append(Rule("lm_head.weight", (config.checkpoint_lm_head_key,), "vocab"))
    n = load_with_rules(model, path, top, DENSE_LAYER, config.num_hidden_layers)
    logger.info("checkpoint loaded path=%s tensors=%d", path, n)


# ------------------------------------------------------------------------- saving
def owner_rank(key: str, tp: int) -> int:
    return zlib.crc32(key.encode()) % tp


def _gather_to(owner: int, t: torch.Tensor, dim: int | None) -> torch.Tensor | None:
    """Gather TP shards along ``dim`` on ``owner`` (None = replicated: owner keeps its copy)."""
    ctx = get_context()
    if ctx.tp_size == 1 or dim is None:
        return t if ctx.tp_rank == owner else None
    parts = [torch.empty_like(t) for _ in range(ctx.tp_size)]
    dist.all_gather(parts, t.contiguous(), group=ctx.tp_group)
    return torch.cat(parts, dim=dim) if ctx.tp_rank == owner else None


def export_rule(param: torch.Tensor, rule: Rule, keys: tuple[str, ...], qkv_meta, vocab: int | None):
    """Yield ``(hf_key, full_tensor_or_None)`` for this rank (None when another rank owns the key)."""
    ctx = get_context()
    tp = ctx.tp_size
    t = param.detach()
    if rule.kind == "replicated":
        yield keys[0], _gather_to(owner_rank(keys[0], tp), t, None)
    elif rule.kind in ("rows", "cols"):
        yield keys[0], _gather_to(owner_rank(keys[0], tp), t, 0 if rule.kind == "rows" else 1)
    elif rule.kind == "vocab":
        full = _gather_to(owner_rank(keys[0], tp), t, 0)
        yield keys[0], (full[:vocab] if (full is not None and vocab) else full)
    elif rule.kind == "merged_rows":
        sizes = getattr(param, "tp_shard", (None, None))[1] or [t.shape[0] // len(keys)] * len(keys)
        off = 0
        for k, n in zip(keys, sizes):
            yield k, _gather_to(owner_rank(k, tp), t[off:off + n], 0)
            off += n
    elif rule.kind == "qkv":
        if len(qkv_meta) > 4:
            raise ValueError("an uneven (padded) head layout is inference-only and cannot be saved")
        hq_rows, hkv, d, rep = qkv_meta
        q_rows = hq_rows * d
        yield keys[0], _gather_to(owner_rank(keys[0], tp), t[:q_rows], 0)
        for j, k in enumerate(keys[1:]):
            part = t[q_rows + j * hkv * d: q_rows + (j + 1) * hkv * d]
            full = _gather_to(owner_rank(k, tp), part, 0)
            if full is not None and rep > 1:
                # replicated kv heads appear `rep` times in the gathered tensor: keep one copy of each
                full = full.view(tp // rep, rep, hkv * d, *full.shape[1:])[:, 0].reshape(-1, *full.shape[1:])
            yield k, full


def save_with_rules(model, path: str, config, top_rules: list[Rule], layer_rules: list[Rule], num_layers: int,
                    source_path: str | None = None, layers_attr: str = "layers",
                    expert_export: Callable | None = None) -> None:
    from safetensors.torch import save_file

    ctx = get_context()
    # expert parallelism: every data-parallel rank owns different experts and writes them to a file of its own;
    # everything else is written by data-parallel rank 0 as usual
    ep = ctx.ep_size > 1 and expert_export is not None
    if ctx.dp_rank != 0 and not ep:
        if ctx.world_size > 1:
            dist.barrier()
        return
    os.makedirs(path, exist_ok=True)
    tensors: dict[str, torch.Tensor] = {}
    experts_only = ep and ctx.dp_rank != 0

    def emit(rule: Rule, obj, fmt: dict):
        try:
            param = _resolve(obj, rule.attr)
        except AttributeError:
            return
        if param is None:
            return
        keys = tuple(k.format(**fmt) for k in rule.keys)
        meta = (getattr(param, "tp_shard", None) or (None, None))[1] if rule.kind == "qkv" else None
        for k, full in export_rule(param, rule, keys, meta, config.vocab_size if rule.kind == "vocab" else None):
            if full is not None:
                tensors[k] = full.to("cpu", copy=True).contiguous()

    if not experts_only:
        for rule in top_rules:
            emit(rule, model, {})
    layers = _resolve(model, layers_attr)
    for i in range(num_layers):
        if not experts_only:
            for rule in layer_rules:
                emit(rule, layers[i], {"layer": i})
        if expert_export is not None:
            tensors.update(expert_export(layers[i], i))
    tp = ctx.tp_size
    # single-writer checkpoints use the plain Hugging Face file name (as ``areno/engine/checkpoints/io.py:610``)
    if ep:
        fname = f"model-{ctx.ep_rank + 1:05d}-of-{ctx.ep_size:05d}.safetensors"
    else:
        fname = "model.safetensors" if tp == 1 else f"model-{ctx.tp_rank + 1:05d}-of-{tp:05d}.safetensors"
    save_file(tensors, os.path.join(path, fname), metadata={"format": "pt"})
    local = {k: fname for k in tensors}
    size = sum(t.numel() * t.element_size() for t in tensors.values())
    if ep:
        maps = [None] * ctx.ep_size
        dist.all_gather_object(maps, (local, size), group=ctx.ep_ctl_group)
    elif tp > 1:
        maps = [None] * tp
        dist.all_gather_object(maps, (local, size), group=ctx.tp_group)
    else:
        maps = [(local, size)]
    if ctx.tp_rank == 0 and ctx.dp_rank == 0:
        weight_map: dict[str, str] = {}
        total = 0
        for m, s in maps:
            weight_map.update(m)
            total += s
        if source_path and os.path.isdir(source_path):
            total += _passthrough_untouched(source_path, path, weight_map)
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total, "areno_checkpoint_writer": "distributed_tp"},
                       "weight_map": dict(sorted(weight_map.items()))}, f, indent=2)
        copy_assets(source_path, path, config)
    if ctx.world_size > 1:
        dist.barrier()


def _passthrough_untouched(source_path: str, out_path: str, weight_map: dict[str, str]) -> int:
    """Tensors of the source checkpoint that the text model does not own (e.g. a vision tower) are
    copied through unchanged into an extra shard.  Returns their size in bytes (counted in ``total_size``)."""
    from safetensors.torch import save_file

    try:
        src = SafetensorsIndex(source_path)
    except (FileNotFoundError, OSError):
        return 0
    extra = {k: src.get(k) for k in src.keys() if k not in weight_map}
    if not extra:
        return 0
    fname = "model-passthrough.safetensors"
    save_file(extra, os.path.join(out_path, fname), metadata={"format": "pt"})
    for k in extra:
        weight_map[k] = fname
    return sum(t.numel() * t.element_size() for t in extra.values())


def copy_assets(source_path: str | None, out_path: str, config=None) -> None:
    if source_path and os.path.isdir(source_path):
        for name in ASSET_FILES:
            src = os.path.join(source_path, name)
            if os.path.exists(src) and not os.path.exists(os.path.join(out_path, name)):
                shutil.copy2(src, os.path.join(out_path, name))
    cfg_out = os.path.join(out_path, "config.json")
    if not os.path.exists(cfg_out) and config is not None:
        with open(cfg_out, "w") as f:
            json.dump(hf_config_from_model_config(config), f, indent=2)


def hf_config_from_model_config(c) -> dict:
    """Minimal HF ``config.json`` for a synthetic model so that a saved directory can be reloaded."""
    out = {
        "model_type": c.model_type, "vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
        "intermediate_size": c.intermediate_size, "num_hidden_layers": c.num_hidden_layers,
        "num_attention_heads": c.num_attention_heads, "num_key_value_heads": c.num_key_value_heads,
        "head_dim": c.head_dim, "rms_norm_eps": c.rms_norm_eps, "rope_theta": c.rope_theta,
        "max_position_embeddings": c.max_position_embeddings, "tie_word_embeddings": c.tie_word_embeddings,
        "attention_bias": c.qkv_bias, "qk_layernorm": c.qk_norm, "hidden_act": c.hidden_act,
        "torch_dtype": str(c.dtype).replace("torch.", ""),
    }
    if c.num_experts:
        out.update(num_experts=c.num_experts, num_experts_per_tok=c.num_experts_per_tok,
                   moe_intermediate_size=c.moe_intermediate_size, norm_topk_prob=c.norm_topk_prob,
                   decoder_sparse_step=(c.extra or {}).get("decoder_sparse_step", 1),
                   mlp_only_layers=(c.extra or {}).get("mlp_only_layers", []))
    return out


def save_dense_checkpoint(model, path: str, config, source_path: str | None = None) -> None:
    top = list(DENSE_TOP)
    if not config.tie_word_embeddings:
        top.append(Rule("lm_head.weight", (config.checkpoint_lm_head_key,), "vocab"))
    save_with_rules(model, path, config, top, DENSE_LAYER, config.num_hidden_layers, source_path)
    logger.info("checkpoint saved path=%s", path)
