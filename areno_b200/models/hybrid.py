"""Hybrid decoder of the Qwen3.5 / MiniCPM-V-4.6 text family: layers are either gated softmax
attention (q/k head norms, partial rotary embedding, sigmoid output gate) or Gated DeltaNet linear
attention (fused q/k/v/z and b/a projections, depthwise causal conv, gated delta rule, RMSNorm with a
SiLU gate), selected per layer by ``cfg.layer_types``.

Counterpart of ``areno/models/qwen3_5/model.py:90-467`` in the reference.  Differences: the q and gate
halves of HF's ``q_proj`` are two projections here (split at load time), linear-attention state lives
in per-slot caches indexed by the engine's slot id instead of ``block_table[:, 0]``, and the
recurrence / conv / gated-norm are this package's CUDA kernels (``ops/linear_attn.py``) instead of FLA.
Tensor parallelism: both kinds of layer shard their heads over the TP group.  A Gated DeltaNet layer keeps
``linear_num_key_heads / tp`` key heads with the value heads that belong to them (value heads are grouped
consecutively per key head, so rank ``r`` owns one contiguous run of each), slices the fused projections, the
depthwise conv filters, ``A_log`` and ``dt_bias`` accordingly, and reduces after ``out_proj``
(reference: ``areno/models/qwen3_5/model.py:90-190`` shards the same tensors).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..engine.config import ModelConfig
from ..ops import gemm, linear_attn as la
from ..parallel import collectives as coll
from ..parallel.context import get_context
from .dense import Attention, DecoderLayer, DenseCausalLM, TrainMeta
from .layers import ColumnParallelLinear, RowParallelLinear, _param


class GatedAttention(Attention):
    """Softmax attention whose output is multiplied by ``sigmoid(gate)`` before ``o_proj``."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__(cfg, layer_idx, dtype, device)
        self.gate = None
        if cfg.attn_output_gate:
            self.gate = ColumnParallelLinear(cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim, False, dtype, device)

    def forward(self, x, positions, meta):
        o = self.attend(x, positions, meta)
        if self.gate is not None:
            o = o * torch.sigmoid(self.gate(x))
        return self.o(o)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        tp = get_context().tp_size
        if cfg.linear_num_key_heads % tp or cfg.linear_num_value_heads % tp:
            raise ValueError(f"linear-attention heads ({cfg.linear_num_key_heads} key, {cfg.linear_num_value_heads} value) "
                             f"must divide tp_size {tp}")
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.hk, self.hv = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp   # local heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.k = cfg.linear_conv_kernel_dim
        h = cfg.hidden_size
        self.in_qkvz = _param((self.conv_dim + self.value_dim, h), dtype, device)   # rows: q | k | v | z
        self.in_ba = _param((2 * self.hv, h), dtype, device)                         # rows: b | a
        self.conv_weight = _param((self.conv_dim, self.k), torch.float32, device)
        self.dt_bias = _param((self.hv,), torch.float32, device)
        self.A_log = _param((self.hv,), torch.float32, device)
        self.norm_weight = _param((self.dv,), torch.float32, device)
        self.norm_weight.tp_replicated_grad = True     # applied to this rank's heads: partial gradient
        # how the local tensors sit in the full ones (used when a TP rollout layout is cut out of a tp=1 replica)
        self.in_qkvz.tp_shard = ("merged", [self.key_dim, self.key_dim, self.value_dim, self.value_dim])
        self.in_ba.tp_shard = ("merged", [self.hv, self.hv])
        self.conv_weight.tp_shard = ("merged", [self.key_dim, self.key_dim, self.value_dim])
        self.dt_bias.tp_shard = ("col", None)
        self.A_log.tp_shard = ("col", None)
        self.out_proj = RowParallelLinear(self.value_dim * tp, h, False, dtype, device)
        self.eps = cfg.rms_norm_eps
        self.scale = self.dk ** -0.5
        self.conv_cache = None    # fp32 [slots, conv_dim, K-1]
        self.state_cache = None   # fp32 [slots, hv, dk, dv]

    # ------------------------------------------------------------------ pieces
    def _gates(self, ba):
        b, a = ba[:, : self.hv].float(), ba[:, self.hv:].float()
        g = -torch.exp(self.A_log.float()) * F.softplus(a + self.dt_bias.float())
        return g.contiguous(), torch.sigmoid(b).contiguous()

    @staticmethod
    def _l2norm(x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + 1e-6)).to(x.dtype)

    def _split(self, mixed):
        t = mixed.shape[0]
        q = mixed[:, : self.key_dim].reshape(t, self.hk, self.dk)
        k = mixed[:, self.key_dim: 2 * self.key_dim].reshape(t, self.hk, self.dk)
        v = mixed[:, 2 * self.key_dim:].reshape(t, self.hv, self.dv)
        return self._l2norm(q), self._l2norm(k), v.contiguous()

    def forward(self, x, positions, meta):
        del positions
        t = x.shape[0]
        x = coll.copy_to_tp(x)   # identity forward, gradient summed over the TP group
        qkvz = gemm.linear(x, self.in_qkvz)
        g, beta = self._gates(gemm.linear(x, self.in_ba))
        conv_in = qkvz[:, : self.conv_dim]
        z = qkvz[:, self.conv_dim:].unflatten(1, (self.hv, self.dv))
        if isinstance(meta, TrainMeta):
            lens = [b - a for a, b in zip(meta.varlen.cu_q_host[:-1], meta.varlen.cu_q_host[1:])]
            mixed = la.conv1d_silu(conv_in, self.conv_weight, lens)
            q, k, v = self._split(mixed)
            o = la.gated_delta_rule_chunked(q, k, v, g, beta, lens, self.scale)
        elif meta.mode == "decode":
            active = meta.seq_lens
            mixed = la.conv1d_silu_decode(conv_in, self.conv_weight, self.conv_cache, active)
            q, k, v = self._split(mixed)
            cu = torch.arange(t + 1, dtype=torch.int32, device=x.device)
            o = self._recurrent(q, k, v, g, beta, [1] * t, cu, None, None, active)
        else:
            lens = [b - a for a, b in zip(meta.varlen.cu_q_host[:-1], meta.varlen.cu_q_host[1:])]
            slots, fresh = meta.seq_slots, meta.seq_fresh
            hist = self.conv_cache.index_select(0, slots.long()) * (1 - fresh.to(torch.float32))[:, None, None]
            mixed = la.conv1d_silu(conv_in, self.conv_weight, lens, hist=hist.contiguous())
            la.conv1d_update_hist(conv_in, meta.varlen.cu_q, slots, fresh, self.conv_cache, self.k)
            q, k, v = self._split(mixed)
            o = self._recurrent(q, k, v, g, beta, lens, meta.varlen.cu_q, slots, fresh, None)
        o = la.rmsnorm_silu_gate(o.contiguous(), z, self.norm_weight, self.eps)
        return self.out_proj(o.reshape(t, self.value_dim))

    def _recurrent(self, q, k, v, g, beta, lens, cu, slots, fresh, active):
        if q.is_cuda:
            qk = torch.stack([q, k], 0).contiguous()  # same row stride for q and k
            return la.gated_delta_rule_recurrent(qk[0], qk[1], v, g, beta, cu, self.scale, state_cache=self.state_cache,
                                                 slots=slots, fresh=fresh, active=active)
        # CPU: the PyTorch recurrence with explicit state hand-over
        n = len(lens)
        slot_ids = list(range(n)) if slots is None else [int(s) for s in slots]
        is_fresh = [False] * n if fresh is None else [bool(f) for f in fresh]
        is_active = [True] * n if active is None else [bool(a > 0) for a in active[:n]]
        states = [torch.zeros_like(self.state_cache[0]) if is_fresh[i] else self.state_cache[slot_ids[i]] for i in range(n)]
        out, finals = la.gated_delta_rule_reference(q, k, v, g, beta, lens, self.scale, states)
        for i in range(n):
            if is_active[i]:
                self.state_cache[slot_ids[i]] = finals[i]
        return out


class HybridDecoderLayer(DecoderLayer):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        kind = cfg.layer_types[layer_idx] if cfg.layer_types else "full_attention"
        mixer = GatedDeltaNet if kind == "linear_attention" else GatedAttention
        attn = mixer(cfg, layer_idx, dtype, device)
        mlp = None
        if cfg.num_experts:
            from .moe import SparseMoeBlock

            mlp = SparseMoeBlock(cfg, dtype, device)
        super().__init__(cfg, layer_idx, dtype, device, mlp=mlp, attn=attn)
        self.kind = kind


class HybridCausalLM(DenseCausalLM):
    def _make_layer(self, i, dtype, device):
        return HybridDecoderLayer(self.cfg, i, dtype, device)

    def _softmax_layers(self):
        return [layer for layer in self.layers if layer.kind != "linear_attention"]

    def _linear_layers(self):
        return [layer for layer in self.layers if layer.kind == "linear_attention"]

    # ------------------------------------------------------------- engine lifecycle
    def kv_cache_bytes_per_page(self, fp8: bool) -> int:
        from ..ops import paged_attention as pa

        layers = self._softmax_layers()
        if not layers:
            return 1
        a = layers[0].attn
        per = a.hkv * pa.PAGE * a.d * (1 if fp8 else 2) * 2
        if fp8:
            per += a.hkv * pa.PAGE * 4 * 2
        return per * len(layers)

    def state_bytes_per_slot(self) -> int:
        total = 0
        for layer in self._linear_layers():
            a = layer.attn
            total += 4 * (a.conv_dim * (a.k - 1) + a.hv * a.dk * a.dv)
        return total

    def allocate_kv_caches(self, num_pages: int, fp8: bool = False, max_slots: int | None = None) -> None:
        from ..ops import paged_attention as pa

        dev = self.embed.weight.device
        for layer in self._softmax_layers():
            a = layer.attn
            a.kv_cache = pa.alloc_kv_cache(num_pages, a.hkv, a.d, dev, fp8)
        slots = int(max_slots or getattr(self, "_max_slots", 0) or 64)
        self._max_slots = slots
        for layer in self._linear_layers():
            a = layer.attn
            a.conv_cache = torch.zeros((slots, a.conv_dim, a.k - 1), dtype=torch.float32, device=dev)
            a.state_cache = torch.zeros((slots, a.hv, a.dk, a.dv), dtype=torch.float32, device=dev)
        self._kv_spec = (num_pages, fp8)

    def set_max_slots(self, max_slots: int) -> None:
        if getattr(self, "_max_slots", 0) < max_slots:
            self._max_slots = int(max_slots)
            self._kv_spec = None  # forces re-allocation with enough state slots

    def kv_caches(self):
        return [layer.attn.kv_cache if layer.kind != "linear_attention" else (layer.attn.conv_cache, layer.attn.state_cache)
                for layer in self.layers]

    def set_kv_caches(self, caches) -> None:
        for layer, c in zip(self.layers, caches):
            if layer.kind == "linear_attention":
                layer.attn.conv_cache, layer.attn.state_cache = c
            else:
                layer.attn.kv_cache = c

    def clear_kv_caches(self) -> None:
        for layer in self.layers:
            if layer.kind == "linear_attention":
                layer.attn.conv_cache = layer.attn.state_cache = None
            else:
                layer.attn.kv_cache = None
        self._kv_spec = None

    def reset_kv_caches(self) -> None:
        """Recurrent state is reset per sequence by the ``fresh`` flag of its first prefill chunk."""
