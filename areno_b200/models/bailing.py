"""Bailing-MoE-Linear-V2 / V2.5 decoder: layers grouped in blocks of ``layer_group_size`` whose last
layer runs softmax attention (grouped-query, or multi-head latent attention when ``kv_lora_rank`` is
set) and whose other layers run decayed linear ("lightning") attention with a per-head, per-layer
slope, a sigmoid-gated group RMSNorm on the attention output and a recurrent state per engine slot.
The feed-forward is dense for the first ``first_k_dense_replace`` layers and a sparse block after
that: sigmoid scores, selection bias, group-limited top-k, renormalised weights times
``routed_scaling_factor``, optional shared experts, and a bias update after every optimizer step that
nudges under-loaded experts up and over-loaded ones down.

Counterpart of ``areno/models/bailing/model.py:92-1233`` in the reference.  Differences: the router,
permute / combine and grouped GEMMs are the device-planned path of ``ops/moe.py`` for training and
inference alike (no separate fused-inference weights to prepare); linear attention is one CUDA scan
kernel with a hand-written backward (``ops/linear_attn.py``) instead of FLA's chunked Triton kernel for
training and ``seg_la`` for inference; recurrent state is indexed by the engine's slot id; latent
attention pads q / k / v with zero channels to the next kernel head size (192 -> 256) instead of
calling flash-attn with unequal q-k and v widths.  All layer kinds shard their heads (and norm groups) over TP.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..engine.config import ModelConfig
from ..ops import attention as attn_ops
from ..ops import gemm, linear_attn as la, moe as moe_ops, paged_attention as pa, rope as rope_ops
from ..parallel import collectives as coll
from ..parallel.context import get_context
from .dense import Attention, DecoderLayer, DenseCausalLM, TrainMeta, _gather_history
from .layers import ColumnParallelLinear, GatedMLP, MergedColumnParallelLinear, RMSNorm, RowParallelLinear, _param
from .moe import Experts


def is_softmax_layer(cfg: ModelConfig, i: int) -> bool:
    """Last layer of every group, plus the tail that does not fill a group
    (``areno/models/bailing/model.py:1361-1373``)."""
    g = max(1, cfg.layer_group_size)
    return (i + 1) % g == 0 or i >= cfg.num_hidden_layers // g * g


def build_slopes(heads: int, layer_idx: int, num_layers: int) -> torch.Tensor:
    """ALiBi-style geometric slopes per head, scaled down linearly with depth
    (``areno/models/bailing/model.py:1376-1413``)."""

    def pow2(m):
        start = 2 ** (-(2 ** -(math.log2(m) - 3)))
        return [start * start ** i for i in range(m)]

    def slopes(n):
        if math.log2(n).is_integer():
            return pow2(n)
        c = 2 ** math.floor(math.log2(n))
        return pow2(c) + slopes(2 * c)[0::2][: n - c]

    layer_scale = 1 + 1e-5 if num_layers <= 1 else 1 - layer_idx / (num_layers - 1) + 1e-5
    return torch.tensor(slopes(heads), dtype=torch.float32) * layer_scale


def _trailing_interleaved_freqs(head_dim: int, rope_dim: int, theta: float, device) -> torch.Tensor:
    """Frequency table for interleaved-pair rotation of the LAST ``rope_dim`` channels of a head: the
    kernels rotate pairs ``(2i, 2i+1)`` of the whole head, pairs in the leading channels get frequency 0."""
    assert rope_dim % 2 == 0 and (head_dim - rope_dim) % 2 == 0
    f = torch.zeros(head_dim // 2, dtype=torch.float32)
    f[(head_dim - rope_dim) // 2:] = theta ** (-torch.arange(0, rope_dim, 2, dtype=torch.float32) / rope_dim)
    return f.to(device)


# ------------------------------------------------------------------------------ softmax attention
class BailingGQAttention(Attention):
    """Fused-QKV grouped-query attention; rotary embedding on the trailing ``qk_rope_head_dim`` channels,
    interleaved pairs (``areno/models/bailing/model.py:722-745``)."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__(cfg, layer_idx, dtype, device)
        self.o = RowParallelLinear(cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size, cfg.use_bias, dtype, device)
        rope_dim = int(cfg.qk_rope_head_dim or cfg.head_dim * cfg.partial_rotary_factor)
        self.rot_dim, self.rope_interleaved = cfg.head_dim, True
        del self.inv_freq
        self.register_buffer("inv_freq", _trailing_interleaved_freqs(cfg.head_dim, rope_dim, cfg.rope_theta, device),
                             persistent=False)


class BailingMLAttention(nn.Module):
    """Multi-head latent attention: per-head queries, keys / values decompressed from a shared low-rank
    projection, one rotary key channel block shared by all heads
    (``areno/models/bailing/model.py:747-763``).  The cache holds the decompressed per-head keys and values."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        ctx = get_context()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.nope = int(cfg.qk_nope_head_dim or cfg.head_dim)
        self.rope = int(cfg.qk_rope_head_dim or cfg.head_dim * cfg.partial_rotary_factor)
        self.vd = int(cfg.v_head_dim or cfg.head_dim)
        self.dqk = self.nope + self.rope
        self.lora = int(cfg.kv_lora_rank)
        need = max(self.dqk, self.vd)
        self.d = next((c for c in (64, 128, 256) if c >= need), None)   # kernel head size after zero padding
        if self.d is None:
            raise ValueError(f"latent attention head size {need} exceeds the largest attention kernel (256)")
        heads = cfg.num_attention_heads
        assert heads % ctx.tp_size == 0
        self.h = heads // ctx.tp_size
        self.hq = self.hkv = self.h
        self.q_proj = ColumnParallelLinear(cfg.hidden_size, heads * self.dqk, False, dtype, device)
        self.kv_a = _param((self.lora + self.rope, cfg.hidden_size), dtype, device)
        self.kv_a.tp_replicated_grad = "same"     # both of its outputs get their gradient summed over TP downstream
        self.kv_a_norm = RMSNorm(self.lora, cfg.rms_norm_eps, dtype, device)
        self.kv_b = ColumnParallelLinear(self.lora, heads * (self.nope + self.vd), False, dtype, device)
        self.o = RowParallelLinear(heads * self.vd, cfg.hidden_size, cfg.use_bias, dtype, device)
        self.scale = self.dqk ** -0.5
        freqs = cfg.rope_theta ** (-torch.arange(0, self.rope, 2, dtype=torch.float32) / self.rope)
        self.register_buffer("inv_freq", freqs.to(device), persistent=False)
        self.kv_cache = None

    def _rotate(self, x, positions):
        return rope_ops.apply_rope(x.clone(memory_format=torch.contiguous_format), positions, rot_dim=self.rope, inv_freq=self.inv_freq, interleaved=True)

    def _project(self, x, positions):
        t, h = x.shape[0], self.h
        q = self.q_proj(x).view(t, h, self.dqk)
        kv_a = gemm.linear(x, self.kv_a)
        # the rotary key block is shared by all heads: each rank back-propagates its own heads' part, copy_to_tp sums them
        k_rope = self._rotate(coll.copy_to_tp(kv_a[:, self.lora:]).reshape(t, 1, self.rope), positions)
        kv = self.kv_b(self.kv_a_norm(kv_a[:, : self.lora].contiguous())).view(t, h, self.nope + self.vd)
        q_rope = self._rotate(q[..., self.nope:], positions)
        pad_qk = q.new_zeros((t, h, self.d - self.dqk))
        q = torch.cat([q[..., : self.nope], q_rope, pad_qk], -1)
        k = torch.cat([kv[..., : self.nope], k_rope.expand(t, h, self.rope), pad_qk], -1)
        v = torch.cat([kv[..., self.nope:], q.new_zeros((t, h, self.d - self.vd))], -1)
        return q, k, v

    def forward(self, x, positions, meta):
        t, h, d = x.shape[0], self.h, self.d
        q, k, v = self._project(x, positions)
        if isinstance(meta, TrainMeta):
            o = attn_ops.varlen_attention(q, k, v, meta.varlen, self.scale, True, 0)
        else:
            kc, vc, ks, vs = self.kv_cache
            qkv = torch.cat([q.reshape(t, h * d), k.reshape(t, h * d), v.reshape(t, h * d)], 1)
            pa.rope_append_kv(qkv, positions, meta.slot_mapping, kc, vc, ks, vs, h, h, d, rot_dim=0)   # already rotated
            q3 = qkv[:, : h * d].unflatten(1, (h, d))
            if meta.mode == "decode":
                o = pa.paged_decode(q3, kc, vc, ks, vs, meta.block_table, meta.seq_lens, self.scale,
                                    max_context=meta.max_context)
            else:
                if meta.has_history:
                    k, v = _gather_history(self.kv_cache, meta, h, d)
                o, _ = attn_ops.attention_forward(q3, k.contiguous(), v.contiguous(), meta.varlen, self.scale, True, 0,
                                                  need_lse=False)
        return self.o(o[..., : self.vd].reshape(t, h * self.vd))


# ------------------------------------------------------------------------------- linear attention
class BailingLinearAttention(nn.Module):
    """Decayed linear attention with q / k head norms, partial rotary embedding (half-split pairs on the
    leading channels), and ``group_rmsnorm(out) * sigmoid(g_proj(x))`` before the output projection
    (``areno/models/bailing/model.py:778-1003``)."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        ctx = get_context()
        tp = ctx.tp_size
        if str((cfg.extra or {}).get("linear_backend", "seg_la")) != "seg_la":
            raise ValueError("Bailing linear attention expects linear_backend='seg_la'")
        self.cfg, self.layer_idx = cfg, layer_idx
        heads = cfg.num_attention_heads
        if heads % tp:
            raise ValueError(f"{heads} attention heads do not divide tp_size {tp}")
        self.h, self.d = heads // tp, cfg.head_dim          # heads of this TP rank
        hd_full = heads * self.d
        hd = self.h * self.d
        # q | k | v are three projections fused into one GEMM, each sharded by heads
        self.qkv = MergedColumnParallelLinear(cfg.hidden_size, [hd_full] * 3, cfg.qkv_bias, dtype, device)
        self.g_proj = ColumnParallelLinear(cfg.hidden_size, hd_full, False, dtype, device)
        self.out_proj = RowParallelLinear(hd_full, cfg.hidden_size, cfg.use_bias, dtype, device)
        groups_full = int(cfg.group_norm_size) if cfg.group_norm_size > 1 else 1
        if hd_full % groups_full != 0:
            raise ValueError(f"hidden width {hd_full} must be divisible by group_norm_size={groups_full}")
        if groups_full % tp:
            raise ValueError(f"group_norm_size {groups_full} must be a multiple of tp_size {tp}: a norm group cannot "
                             "straddle two ranks")
        self.groups = groups_full // tp
        self.g_norm_weight = _param((hd,), torch.float32, device)      # viewed as [groups, hd / groups]; this rank's channels
        self.g_norm_weight.tp_shard = ("col", None)
        self.q_norm = RMSNorm(self.d, cfg.rms_norm_eps, torch.float32, device) if cfg.qk_norm else None
        self.k_norm = RMSNorm(self.d, cfg.rms_norm_eps, torch.float32, device) if cfg.qk_norm else None
        for n in (self.q_norm, self.k_norm):
            if n is not None:
                n.weight.tp_replicated_grad = True     # local heads only
        self.rot = int(self.d * cfg.partial_rotary_factor)
        self.silu = bool(cfg.linear_silu)
        self.eps = cfg.rms_norm_eps
        self.scale = self.d ** -0.5
        slopes = build_slopes(heads, layer_idx, cfg.num_hidden_layers)[ctx.tp_rank * self.h:(ctx.tp_rank + 1) * self.h]
        self.register_buffer("slope", slopes.contiguous().to(device), persistent=False)
        self.state_cache = None   # fp32 [slots, heads, d, d]

    # pieces ------------------------------------------------------------------
    def _qkv_train(self, qkv, positions):
        t, h, d = qkv.shape[0], self.h, self.d
        q, k, v = (qkv[:, i * h * d:(i + 1) * h * d].reshape(t, h, d) for i in range(3))
        if self.q_norm is not None:
            q = attn_ops.head_rmsnorm(q, self.q_norm.weight, self.eps)
            k = attn_ops.head_rmsnorm(k, self.k_norm.weight, self.eps)
        else:
            q, k = q.contiguous(), k.contiguous()      # private copies: the rotation below works in place
        if self.rot > 0:
            q = rope_ops.apply_rope(q, positions, self.cfg.rope_theta, self.rot)
            k = rope_ops.apply_rope(k, positions, self.cfg.rope_theta, self.rot)
        return q, k, v.contiguous()

    def _qkv_infer(self, qkv, positions):
        t, h, d = qkv.shape[0], self.h, self.d
        q, k, v = (qkv[:, i * h * d:(i + 1) * h * d].unflatten(1, (h, d)) for i in range(3))
        for x3, norm in ((q, self.q_norm), (k, self.k_norm)):
            if norm is not None:
                if x3.is_cuda:
                    attn_ops._headnorm_fwd(x3, norm.weight, 0.0, x3, self.eps)
                else:
                    x3.copy_(attn_ops._headnorm_reference(x3, norm.weight, self.eps, 0.0))
            if self.rot > 0:
                r = rope_ops.apply_rope(x3, positions, self.cfg.rope_theta, self.rot)
                if r is not x3:
                    x3.copy_(r)
        return q, k, v

    def forward(self, x, positions, meta):
        t, h, d = x.shape[0], self.h, self.d
        qkv = self.qkv(x)
        if self.silu:
            qkv = F.silu(qkv)
        if isinstance(meta, TrainMeta):
            q, k, v = self._qkv_train(qkv, positions)
            lens = [b - a for a, b in zip(meta.varlen.cu_q_host[:-1], meta.varlen.cu_q_host[1:])]
            o = la.lightning_attention(q, k, v, self.slope, lens, self.scale, cu=meta.varlen.cu_q)
        else:
            q, k, v = self._qkv_infer(qkv, positions)
            if meta.mode == "decode":
                cu = torch.arange(t + 1, dtype=torch.int32, device=x.device)
                o = self._scan(q, k, v, [1] * t, cu, None, None, meta.seq_lens)
            else:
                lens = [b - a for a, b in zip(meta.varlen.cu_q_host[:-1], meta.varlen.cu_q_host[1:])]
                o = self._scan(q, k, v, lens, meta.varlen.cu_q, meta.seq_slots, meta.seq_fresh, None)
        gate = self.g_proj(x)
        o = la.group_rmsnorm_sigmoid_gate(o.reshape(t, h * d).contiguous(), gate,
                                          self.g_norm_weight.view(self.groups, -1), self.eps)
        return self.out_proj(o)

    def _scan(self, q, k, v, lens, cu, slots, fresh, active):
        if q.is_cuda:
            return la.lightning_recurrent(q, k, v, self.slope, cu, self.scale, state_cache=self.state_cache, slots=slots,
                                          fresh=fresh, active=active)
        n = len(lens)
        slot_ids = list(range(n)) if slots is None else [int(s) for s in slots]
        is_fresh = [False] * n if fresh is None else [bool(f) for f in fresh]
        is_active = [True] * n if active is None else [bool(a > 0) for a in active[:n]]
        states = [None if is_fresh[i] else self.state_cache[slot_ids[i]] for i in range(n)]
        out, finals = la.lightning_attention_reference(q, k, v, self.slope, lens, self.scale, states)
        for i in range(n):
            if is_active[i]:
                self.state_cache[slot_ids[i]] = finals[i]
        return out


# ------------------------------------------------------------------------------------------ MoE
class BailingGate(nn.Module):
    """Router: fp32 projection, sigmoid scores, selection bias, group-limited top-k; no gradient flows
    through the routing weights (``areno/models/bailing/model.py:111-198``)."""

    def __init__(self, cfg: ModelConfig, device):
        super().__init__()
        if cfg.score_function != "sigmoid":
            raise ValueError(f"BailingGate only supports sigmoid scoring, got {cfg.score_function!r}")
        if not cfg.moe_router_enable_expert_bias:
            raise ValueError("BailingGate requires expert bias for biased grouped top-k")
        if not cfg.norm_topk_prob:
            raise ValueError("BailingGate requires norm_topk_prob=True")
        self.k, self.e = cfg.num_experts_per_tok, int(cfg.num_experts)
        self.n_group, self.topk_group = cfg.n_group, cfg.topk_group
        self.scaling = float(cfg.routed_scaling_factor)
        self.rate = float(cfg.moe_router_bias_update_rate)
        self.weight = _param((self.e, cfg.hidden_size), cfg.moe_router_dtype, device)
        self.weight.tp_replicated_grad = True
        self.register_buffer("tokens_per_expert", torch.zeros(self.e, dtype=torch.float32, device=device), persistent=False)
        self.register_buffer("expert_bias", torch.zeros(self.e, dtype=torch.float32, device=device), persistent=False)

    def forward(self, x):
        logits = F.linear(x.to(self.weight.dtype), self.weight)
        w, ids = moe_ops.grouped_sigmoid_topk(logits, self.expert_bias, self.n_group, self.topk_group, self.k, True,
                                              self.scaling)
        if torch.is_grad_enabled():
            flat = ids.reshape(-1).long()
            self.tokens_per_expert.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.float32))
        return w, ids

    @torch.no_grad()
    def finalize_expert_bias(self, dp_group=None) -> None:
        """Sum the step's token counts over data-parallel replicas, move each expert's bias one signed step
        toward the mean load, re-centre to zero mean, reset the counter."""
        import torch.distributed as dist

        counts = self.tokens_per_expert
        if dp_group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(dp_group) > 1:
            dist.all_reduce(counts, group=dp_group)
        if self.rate != 0.0:
            self.expert_bias.add_(torch.sign(counts.mean() - counts) * self.rate)
            self.expert_bias.sub_(self.expert_bias.mean())
        counts.zero_()


class BailingSparseMoeBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.gate = BailingGate(cfg, device)
        self.experts = Experts(cfg, dtype, device)
        self.shared = None
        if cfg.num_shared_experts:
            self.shared = GatedMLP(cfg.hidden_size, cfg.moe_intermediate_size * int(cfg.num_shared_experts), cfg.hidden_act,
                                   False, dtype, device)
        self.last_counts = None

    def forward(self, x):
        x_tp = coll.copy_to_tp(x)      # experts are sharded over TP: sum the token gradient of the ranks' routes
        w, ids = self.gate(x_tp)
        out, plan = self.experts(x_tp, w, ids)
        self.last_counts = plan.counts
        if self.shared is not None:
            out = out + self.shared(x)
        return out


# ---------------------------------------------------------------------------------------- model
class BailingDecoderLayer(DecoderLayer):
    def __init__(self, cfg: ModelConfig, i: int, dtype, device):
        kind = "attention" if is_softmax_layer(cfg, i) else "linear_attention"
        if kind == "linear_attention":
            attn = BailingLinearAttention(cfg, i, dtype, device)
        elif cfg.kv_lora_rank is not None:
            attn = BailingMLAttention(cfg, i, dtype, device)
        else:
            attn = BailingGQAttention(cfg, i, dtype, device)
        sparse = cfg.num_experts is not None and i >= cfg.first_k_dense_replace
        mlp = BailingSparseMoeBlock(cfg, dtype, device) if sparse else None
        super().__init__(cfg, i, dtype, device, mlp=mlp, attn=attn)
        self.kind = kind


class BailingCausalLM(DenseCausalLM):
    def _make_layer(self, i, dtype, device):
        return BailingDecoderLayer(self.cfg, i, dtype, device)

    def _softmax_layers(self):
        return [layer for layer in self.layers if layer.kind == "attention"]

    def _linear_layers(self):
        return [layer for layer in self.layers if layer.kind == "linear_attention"]

    def finalize_router_expert_bias(self, tp_group=None, dp_group=None) -> None:
        del tp_group
        for layer in self.layers:
            if isinstance(layer.mlp, BailingSparseMoeBlock):
                layer.mlp.gate.finalize_expert_bias(dp_group)

    # ------------------------------------------------------------- engine lifecycle
    def kv_cache_bytes_per_page(self, fp8: bool) -> int:
        total = 0
        for layer in self._softmax_layers():
            a = layer.attn
            per = a.hkv * pa.PAGE * a.d * (1 if fp8 else 2) * 2
            if fp8:
                per += a.hkv * pa.PAGE * 4 * 2
            total += per
        return max(total, 1)

    def state_bytes_per_slot(self) -> int:
        return sum(4 * layer.attn.h * layer.attn.d * layer.attn.d for layer in self._linear_layers())

    def allocate_kv_caches(self, num_pages: int, fp8: bool = False, max_slots: int | None = None) -> None:
        dev = self.embed.weight.device
        for layer in self._softmax_layers():
            a = layer.attn
            a.kv_cache = pa.alloc_kv_cache(num_pages, a.hkv, a.d, dev, fp8)
        slots = int(max_slots or getattr(self, "_max_slots", 0) or 64)
        self._max_slots = slots
        for layer in self._linear_layers():
            a = layer.attn
            a.state_cache = torch.zeros((slots, a.h, a.d, a.d), dtype=torch.float32, device=dev)
        self._kv_spec = (num_pages, fp8)

    def set_max_slots(self, max_slots: int) -> None:
        if getattr(self, "_max_slots", 0) < max_slots:
            self._max_slots = int(max_slots)
            self._kv_spec = None   # forces re-allocation with enough state slots

    def kv_caches(self):
        return [layer.attn.kv_cache if layer.kind == "attention" else layer.attn.state_cache for layer in self.layers]

    def set_kv_caches(self, caches) -> None:
        for layer, c in zip(self.layers, caches):
            if layer.kind == "attention":
                layer.attn.kv_cache = c
            else:
                layer.attn.state_cache = c

    def clear_kv_caches(self) -> None:
        for layer in self.layers:
            if layer.kind == "attention":
                layer.attn.kv_cache = None
            else:
                layer.attn.state_cache = None
        self._kv_spec = None

    def reset_kv_caches(self) -> None:
        """Recurrent state is reset per sequence by the ``fresh`` flag of its first prefill chunk."""
