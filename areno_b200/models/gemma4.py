"""Gemma-4 text decoder.

Per-layer attention type (``full_attention`` / ``sliding_attention``) selects head dim, KV-head
count, RoPE base / rotated fraction and the sliding window; q / k / v get per-head RMSNorm (v
without a learned scale); the softmax scale is 1; the last ``num_kv_shared_layers`` layers project
only queries and attend to the K / V of the nearest earlier layer of their type; blocks use
sandwich norms, an optional mixture-of-experts branch in parallel with the dense GeGLU MLP, optional
per-layer-input embeddings (PLE) and a per-layer output scalar; embeddings are scaled by
``sqrt(hidden)`` and the final logits are soft-capped.

Counterpart of ``areno/models/gemma4/model.py:64-760`` in the reference.  Training composes
differentiable kernels (head norm, RoPE, varlen attention); inference uses the in-place fused RoPE +
KV-append and the paged decode kernel, with KV-shared layers bound to their source layer's cache.
"""

from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..engine.config import ModelConfig
from ..ops import activation, attention as attn_ops, gemm, moe as moe_ops, paged_attention as pa, rope as rope_ops
from ..parallel import collectives as coll
from ..parallel.context import get_context
from .dense import CausalLMOutput, DenseCausalLM, InferMeta, TrainMeta, _gather_history
from .layers import (GatedMLP, QKVParallelLinear, RMSNorm, RowParallelLinear, VocabParallelEmbedding, _param)


def layer_type(cfg: ModelConfig, i: int) -> str:
    return cfg.layer_types[i] if cfg.layer_types else "full_attention"


def kv_source_layer(cfg: ModelConfig, i: int) -> int | None:
    """Index of the layer whose K / V layer ``i`` reuses, or None when it projects its own."""
    first_shared = cfg.num_hidden_layers - cfg.num_kv_shared_layers
    if cfg.num_kv_shared_layers <= 0 or i < first_shared:
        return None
    kind = layer_type(cfg, i)
    for j in range(first_shared - 1, -1, -1):
        if layer_type(cfg, j) == kind:
            return j
    raise ValueError(f"KV-shared layer {i} has no earlier {kind!r} layer")


def _rope_inv_freq(head_dim: int, theta: float, partial: float, device) -> torch.Tensor:
    """Frequencies over the FULL head (pairs i, i + head_dim/2); channels past the rotated fraction get
    frequency 0, i.e. the identity rotation."""
    rot_pairs = int(head_dim * partial) // 2
    inv = 1.0 / (theta ** (torch.arange(0, 2 * rot_pairs, 2, dtype=torch.float32) / head_dim))
    pad = head_dim // 2 - rot_pairs
    if pad > 0:
        inv = torch.cat([inv, torch.zeros(pad)])
    return inv.to(device)


class Gemma4Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        kind = layer_type(cfg, layer_idx)
        sliding = kind == "sliding_attention"
        self.d = int(cfg.swa_head_dim) if sliding and cfg.swa_head_dim else int(cfg.head_dim)
        kv_heads = int(cfg.swa_num_key_value_heads) if sliding and cfg.swa_num_key_value_heads else int(cfg.num_key_value_heads)
        self.qkv = QKVParallelLinear(cfg.hidden_size, cfg.num_attention_heads, kv_heads, self.d, cfg.qkv_bias, dtype, device)
        self.hq, self.hkv = self.qkv.hq, self.qkv.hkv
        self.o = RowParallelLinear(cfg.num_attention_heads * self.d, cfg.hidden_size, cfg.qkv_bias, dtype, device)
        self.q_norm = RMSNorm(self.d, cfg.rms_norm_eps, torch.float32, device)
        self.k_norm = RMSNorm(self.d, cfg.rms_norm_eps, torch.float32, device)
        self.q_norm.weight.tp_replicated_grad = self.k_norm.weight.tp_replicated_grad = True   # local heads only
        self.v_norm = bool(cfg.v_norm)
        self.window = int(cfg.sliding_window) if sliding and cfg.sliding_window else 0   # inclusive of the current token
        self.scale = float(cfg.attention_softmax_scale or self.d ** -0.5)
        params = (cfg.rope_parameters or {}).get(kind, {})
        theta = float(params.get("rope_theta", cfg.rope_theta))
        partial = float(params.get("partial_rotary_factor", cfg.partial_rotary_factor))
        self.register_buffer("inv_freq", _rope_inv_freq(self.d, theta, partial, device), persistent=False)
        self.register_buffer("unit_scale", torch.ones(self.d, dtype=torch.float32, device=device), persistent=False)
        self.kv_source = kv_source_layer(cfg, layer_idx)
        self.kv_cache = None
        self.eps = cfg.rms_norm_eps

    # ---------------------------------------------------------------- training
    def _train(self, qkv, positions, meta: TrainMeta, shared_kv):
        t = qkv.shape[0]
        hq, hkv, d = self.hq, self.hkv, self.d
        q = attn_ops.head_rmsnorm(qkv[:, : hq * d].reshape(t, hq, d), self.q_norm.weight, self.eps)
        q = rope_ops.apply_rope(q, positions, inv_freq=self.inv_freq, rot_dim=d)
        if shared_kv is not None:
            k, v = shared_kv
            share = None
        else:
            k = attn_ops.head_rmsnorm(qkv[:, hq * d:(hq + hkv) * d].reshape(t, hkv, d), self.k_norm.weight, self.eps)
            k = rope_ops.apply_rope(k, positions, inv_freq=self.inv_freq, rot_dim=d)
            v = qkv[:, (hq + hkv) * d:].reshape(t, hkv, d)
            if self.v_norm:
                v = attn_ops.head_rmsnorm(v, self.unit_scale, self.eps)
            share = (k, v)
        o = attn_ops.varlen_attention(q.contiguous(), k.contiguous(), v.contiguous(), meta.varlen, self.scale, True, self.window)
        return o.reshape(t, hq * d), share

    # --------------------------------------------------------------- inference
    def _norm_inplace(self, x3, w):
        ww = w if w is not None else self.unit_scale
        if x3.is_cuda:
            attn_ops._headnorm_fwd(x3, ww, 0.0, x3, self.eps)
        else:
            x3.copy_(attn_ops._headnorm_reference(x3, ww, self.eps, 0.0))

    def _infer(self, qkv, positions, meta: InferMeta):
        t = qkv.shape[0]
        hq, hkv, d = self.hq, self.hkv, self.d
        q3 = qkv[:, : hq * d].unflatten(1, (hq, d))
        self._norm_inplace(q3, self.q_norm.weight)
        kc, vc, ks, vs = self.kv_cache
        if self.kv_source is None:
            self._norm_inplace(qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d)), self.k_norm.weight)
            if self.v_norm:
                self._norm_inplace(qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d)), None)
            pa.rope_append_kv(qkv, positions, meta.slot_mapping, kc, vc, ks, vs, hq, hkv, d, rot_dim=d, inv_freq=self.inv_freq)
        else:
            # queries only; keys / values were written by the source layer earlier in this forward pass
            q_rot = rope_ops.apply_rope(q3.contiguous(), positions, inv_freq=self.inv_freq, rot_dim=d) if qkv.is_cuda \
                else rope_ops.rope_reference(q3, positions, 0.0, d, self.inv_freq)
            q3 = q_rot
        if meta.mode == "decode":
            out = pa.paged_decode(q3, kc, vc, ks, vs, meta.block_table, meta.seq_lens, self.scale,
                                  max_context=meta.max_context, window=self.window)
            return out.reshape(t, hq * d)
        if meta.has_history or self.kv_source is not None:
            k, v = self._cached_kv(meta, hkv, d)
        else:
            k = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
            v = qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d))
        o, _ = attn_ops.attention_forward(q3, k, v, meta.varlen, self.scale, True, self.window, need_lse=False)
        return o.reshape(t, hq * d)

    def _cached_kv(self, meta: InferMeta, hkv: int, d: int):
        if meta.has_history:
            return _gather_history(self.kv_cache, meta, hkv, d)
        slots = meta.slot_mapping.long()
        fake = dataclasses.replace(meta, history=slots)
        return _gather_history(self.kv_cache, fake, hkv, d)

    def forward(self, x, positions, meta, shared_kv=None):
        qkv = self.qkv(x)
        if isinstance(meta, TrainMeta):
            o, share = self._train(qkv, positions, meta, shared_kv)
        else:
            o, share = self._infer(qkv, positions, meta), None
        return self.o(o), share


class ReplicatedLinear(nn.Module):
    """A projection every TP rank holds whole.  ``grad``: ``"same"`` when all ranks compute the same gradient (the
    projection sits on the replicated residual stream), ``True`` when each rank only sees the part that flows through
    its own experts (the router) and the trainer sums them."""

    def __init__(self, in_features: int, out_features: int, dtype, device, grad="same"):
        super().__init__()
        self.weight = _param((out_features, in_features), dtype, device)
        self.weight.tp_replicated_grad = grad

    def forward(self, x):
        return gemm.linear(x, self.weight)


class Gemma4Router(nn.Module):
    """Scale-free RMSNorm, learned per-channel scale times ``hidden ** -0.5``, projection to experts."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, with_scale=False)
        self.scale = _param((cfg.hidden_size,), torch.float32, device)
        self.scale.tp_replicated_grad = True
        self.proj = ReplicatedLinear(cfg.hidden_size, int(cfg.num_experts), dtype, device, grad=True)
        self.root = cfg.hidden_size ** -0.5

    def forward(self, x):
        h = self.norm(x)
        h = h * (self.scale.to(h.dtype) * self.root)
        return self.proj(h)


class Gemma4Moe(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        ctx = get_context()
        e = int(cfg.num_experts)
        assert e % ctx.tp_size == 0
        self.e_local, self.e_lo = e // ctx.tp_size, ctx.tp_rank * (e // ctx.tp_size)
        self.k, self.renorm = cfg.num_experts_per_tok, cfg.norm_topk_prob
        self.inter = cfg.moe_intermediate_size
        self.per_expert_scale = _param((e,), torch.float32, device)
        self.per_expert_scale.tp_replicated_grad = True
        self.gate_up = _param((self.e_local, 2 * self.inter, cfg.hidden_size), dtype, device)
        self.down = _param((self.e_local, cfg.hidden_size, self.inter), dtype, device)
        self.gate_up.tp_shard = ("col", None)
        self.down.tp_shard = ("col", None)

    def forward(self, x, router_logits):
        w, ids = moe_ops.topk_softmax(router_logits.float(), self.k, self.renorm)
        w = w * self.per_expert_scale[ids.long()]
        plan = moe_ops.align(ids, self.e_lo, self.e_local)
        xs = moe_ops.permute(x, plan)
        a = activation.gelu_tanh_and_mul(moe_ops.grouped_linear(xs, self.gate_up, plan))
        ys = moe_ops.grouped_linear(a, self.down, plan)
        return coll.reduce_from_tp(moe_ops.combine(ys, plan, w))


class Gemma4DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, i: int, dtype, device):
        super().__init__()
        h, eps = cfg.hidden_size, cfg.rms_norm_eps
        self.attn = Gemma4Attention(cfg, i, dtype, device)
        first_shared = cfg.num_hidden_layers - cfg.num_kv_shared_layers
        wide = cfg.use_double_wide_mlp and cfg.num_kv_shared_layers > 0 and i >= first_shared
        self.mlp = GatedMLP(h, cfg.intermediate_size * (2 if wide else 1), "gelu_tanh", False, dtype, device)
        norm = lambda: RMSNorm(h, eps, torch.float32, device)
        self.input_norm, self.post_attn_norm, self.pre_ff_norm, self.post_ff_norm = norm(), norm(), norm(), norm()
        self.router = self.moe = self.pre_ff_norm_2 = self.post_ff_norm_1 = self.post_ff_norm_2 = None
        if cfg.enable_moe_block:
            self.router = Gemma4Router(cfg, dtype, device)
            self.moe = Gemma4Moe(cfg, dtype, device)
            self.pre_ff_norm_2, self.post_ff_norm_1, self.post_ff_norm_2 = norm(), norm(), norm()
        self.ple = cfg.hidden_size_per_layer_input
        self.ple_gate = self.ple_proj = self.post_ple_norm = None
        if self.ple > 0:
            self.ple_gate = ReplicatedLinear(h, self.ple, dtype, device)
            self.ple_proj = ReplicatedLinear(self.ple, h, dtype, device)
            self.post_ple_norm = RMSNorm(h, eps, torch.float32, device)
        self.register_buffer("layer_scalar", torch.ones(1, dtype=torch.float32, device=device), persistent=True)

    def forward(self, x, positions, meta, per_layer_input=None, shared_kv=None):
        a, share = self.attn(self.input_norm(x), positions, meta, shared_kv)
        x = x + self.post_attn_norm(a)
        dense = self.mlp(self.pre_ff_norm(x))
        if self.moe is not None:
            # experts are sharded over TP: each rank back-propagates its own routes into the token and the router,
            # copy_to_tp sums those parts (identity in forward)
            expert_in = coll.copy_to_tp(self.pre_ff_norm_2(x))
            router_in = coll.copy_to_tp(x)
            routed = self.moe(expert_in, self.router(router_in))
            ff = self.post_ff_norm_1(dense) + self.post_ff_norm_2(routed)
        else:
            ff = dense
        x = x + self.post_ff_norm(ff)
        if per_layer_input is not None:
            gated = activation.gelu_tanh_and_mul(torch.cat([self.ple_gate(x), per_layer_input], dim=-1))
            x = x + self.post_ple_norm(self.ple_proj(gated))
        return x * self.layer_scalar.to(x.dtype), share


class Gemma4CausalLM(DenseCausalLM):
    supports_sequence_parallel = False     # own layer loop (KV sharing, per-layer inputs): activations stay replicated

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: torch.dtype | None = None):
        cfg = dataclasses.replace(cfg, embed_scale=math.sqrt(cfg.hidden_size))
        super().__init__(cfg, device=device, dtype=dtype)
        dtype = dtype or cfg.dtype
        self.ple = cfg.hidden_size_per_layer_input
        if self.ple > 0:
            n = cfg.num_hidden_layers
            self.ple_vocab = int(cfg.vocab_size_per_layer_input or cfg.vocab_size)
            self.embed_per_layer = VocabParallelEmbedding(self.ple_vocab, n * self.ple, dtype, device, math.sqrt(self.ple))
            self.per_layer_model_projection = ReplicatedLinear(cfg.hidden_size, n * self.ple, dtype, device)
            self.per_layer_projection_norm = RMSNorm(self.ple, cfg.rms_norm_eps, torch.float32, device)

    def _make_layer(self, i, dtype, device):
        return Gemma4DecoderLayer(self.cfg, i, dtype, device)

    def _per_layer_inputs(self, hidden, ids):
        if self.ple <= 0:
            return None
        n = self.cfg.num_hidden_layers
        t = ids.shape[0]
        safe = torch.where((ids >= 0) & (ids < self.ple_vocab), ids, torch.zeros_like(ids))
        emb = self.embed_per_layer(safe).reshape(t, n, self.ple)
        proj = self.per_layer_model_projection(hidden) * (self.cfg.hidden_size ** -0.5)
        proj = self.per_layer_projection_norm(proj.reshape(t * n, self.ple)).reshape(t, n, self.ple)
        return (proj + emb) * (2.0 ** -0.5)

    def forward(self, input_ids, position_ids, meta) -> CausalLMOutput:
        ids = input_ids.reshape(-1)
        positions = position_ids.reshape(-1)
        if positions.dtype != torch.int32:
            positions = positions.to(torch.int32)
        x = self.embed(ids)
        ple = self._per_layer_inputs(x, ids)
        use_ckpt = isinstance(meta, TrainMeta) and meta.activation_checkpointing and torch.is_grad_enabled()
        shared: dict[int, tuple] = {}
        sources = {layer.attn.kv_source for layer in self.layers if layer.attn.kv_source is not None}
        for i, layer in enumerate(self.layers):
            pli = ple[:, i, :].contiguous() if ple is not None else None
            src = layer.attn.kv_source
            kv = shared.get(src) if src is not None else None
            if use_ckpt and src is None and i not in sources:
                x, share = checkpoint(layer, x, positions, meta, pli, None, use_reentrant=False)
            else:
                x, share = layer(x, positions, meta, pli, kv)
            if share is not None and i in sources:
                shared[i] = share
        h = self.norm(x)
        out = CausalLMOutput(hidden_states=h)
        if isinstance(meta, InferMeta):
            rows = h if meta.logit_rows is None else h.index_select(0, meta.logit_rows)
            out.logits_shard = self.compute_logits(rows, out_dtype=torch.float32)
        return out

    # ------------------------------------------------------------- engine lifecycle
    def _own_cache_layers(self):
        return [layer for layer in self.layers if layer.attn.kv_source is None]

    def kv_cache_bytes_per_page(self, fp8: bool) -> int:
        total = 0
        for layer in self._own_cache_layers():
            a = layer.attn
            per = a.hkv * pa.PAGE * a.d * (1 if fp8 else 2) * 2
            if fp8:
                per += a.hkv * pa.PAGE * 4 * 2
            total += per
        return total

    def allocate_kv_caches(self, num_pages: int, fp8: bool = False) -> None:
        dev = self.embed.weight.device
        for layer in self._own_cache_layers():
            a = layer.attn
            a.kv_cache = pa.alloc_kv_cache(num_pages, a.hkv, a.d, dev, fp8)
        for layer in self.layers:
            if layer.attn.kv_source is not None:
                layer.attn.kv_cache = self.layers[layer.attn.kv_source].attn.kv_cache
        self._kv_spec = (num_pages, fp8)

    def set_kv_caches(self, caches) -> None:
        for layer, c in zip(self.layers, caches):
            layer.attn.kv_cache = c
        for layer in self.layers:
            if layer.attn.kv_source is not None:
                layer.attn.kv_cache = self.layers[layer.attn.kv_source].attn.kv_cache
