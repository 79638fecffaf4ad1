"""Pre-norm decoder-only transformer (Llama / Qwen2.5 / Qwen3 dense families).

One module serves three execution modes selected by the meta object:

* ``TrainMeta``  - packed variable-length batch, autograd on, optional per-layer activation
  checkpointing; returns final hidden states (the LM head is applied chunk-wise by the
  log-prob head so ``[T, vocab]`` logits are never resident);
* ``InferMeta(prefill)`` - packed prompts; K/V are rotated, appended to the paged cache and
  attended in one pass;
* ``InferMeta(decode)``  - one token per running sequence against the paged cache; every shape
  is static so the step is captured in a CUDA graph.

Architecture and lifecycle protocol follow ``areno/models/qwen3/model.py:48-72,234-369`` and
``areno/models/llama/model.py`` of the reference; the kernels underneath are this package's own.
"""

from __future__ import annotations

import dataclasses
import os
import zlib
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..engine.config import ModelConfig
from ..ops import attention as attn_ops
from ..ops import gemm, paged_attention as pa
from ..ops.attention import VarlenMeta
from ..parallel import collectives as coll
from ..parallel.context import get_context
from ..parallel.symm import TpPartial
from .layers import (GatedMLP, QKVParallelLinear, RMSNorm, RowParallelLinear, VocabParallelEmbedding,
                     VocabParallelLMHead)


# ARENO_FUSE_QKV_DECODE=0 falls back to the separate fold / head-norm / rope-append kernels (for A/B timing).
_FUSE_QKV_DECODE = os.environ.get("ARENO_FUSE_QKV_DECODE", "1") != "0"


@dataclass
class TrainMeta:
    varlen: VarlenMeta
    activation_checkpointing: bool = True
    packed: bool = True
    checkpoint_layers: int | None = None   # recompute only the first N layers (None = every layer)
    # called with a layer index from backward once that layer's parameter gradients are final (all later
    # layers finished before it); the trainer uses it to start reducing gradient buckets during backward
    layer_grad_hook: Any = None
    # Megatron-style sequence parallelism over the TP group: activations between the TP seams are sharded by tokens
    # (norms, residual adds and dropout-free element-wise work run on 1 / tp of the rows; all-reduces become
    # all-gather + reduce-scatter).  Ignored at tp_size 1.
    sequence_parallel: bool = False


@dataclass
class InferMeta:
    mode: str                                   # "prefill" | "decode"
    slot_mapping: torch.Tensor                  # int32 [T]: cache slot of every input token (-1 = skip)
    varlen: VarlenMeta | None = None            # prefill: q = new tokens, k = cached + new tokens
    block_table: torch.Tensor | None = None     # int32 [B, max_pages]
    seq_lens: torch.Tensor | None = None        # int32 [B]: context length including the new token(s)
    max_context: int | None = None
    logit_rows: torch.Tensor | None = None      # prefill: row indices whose logits are needed
    has_history: bool = False                   # prefill chunk continues sequences with cached tokens
    history: Any = None                         # (page index tensor, lengths) used to gather cached K/V
    seq_slots: torch.Tensor | None = None       # prefill: int32 [num_seqs] engine slot of every packed sequence
    seq_fresh: torch.Tensor | None = None       # prefill: int32 [num_seqs] 1 when the chunk starts its sequence


@dataclass
class CausalLMOutput:
    logits_shard: torch.Tensor | None = None
    hidden_states: torch.Tensor | None = None
    values: torch.Tensor | None = None
    aux: dict = field(default_factory=dict)


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.d = cfg.head_dim
        self.qkv = QKVParallelLinear(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                     cfg.qkv_bias, dtype, device)
        self.hq, self.hkv = self.qkv.hq, self.qkv.hkv
        o_range = None
        if cfg.num_attention_heads % get_context().tp_size != 0:
            # padded heads (inference-only layout): the projection reads this rank's real heads, padding columns are zero
            o_range = (self.hq * cfg.head_dim, self.qkv.q_lo * cfg.head_dim, self.qkv.q_n * cfg.head_dim)
        self.o = RowParallelLinear(cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size, False, dtype, device,
                                   in_range=o_range)
        self.q_norm = self.k_norm = None
        if cfg.qk_norm:
            self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device, cfg.norm_weight_offset)
            self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device, cfg.norm_weight_offset)
            # per-head norms act on this rank's heads only: each rank holds a part of the gradient
            self.q_norm.weight.tp_replicated_grad = True
            self.k_norm.weight.tp_replicated_grad = True
        self.scale = cfg.attention_softmax_scale or cfg.head_dim ** -0.5
        # rotary layout; subclasses may install their own frequency table (e.g. rotation of the trailing channels)
        self.rot_dim, self.rope_interleaved, self.inv_freq = cfg.rotary_dim, cfg.rope_interleaved, None
        self.window = 0
        if cfg.sliding_window and cfg.layer_types is not None and cfg.layer_types[layer_idx] == "sliding_attention":
            self.window = int(cfg.sliding_window)
        self.kv_cache = None  # (k_cache, v_cache, k_scale, v_scale)

    def forward(self, x, positions, meta):
        return self.o(self.attend(x, positions, meta))

    def attend(self, x, positions, meta):
        """Attention output ``[T, hq * d]`` before the output projection."""
        cfg = self.cfg
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        if isinstance(meta, TrainMeta):
            return attn_ops.qkv_attention(
                self.qkv(x), positions, meta.varlen, self.hq, self.hkv, self.d, scale=self.scale, theta=cfg.rope_theta,
                rot_dim=self.rot_dim, inv_freq=self.inv_freq, interleaved=self.rope_interleaved, causal=True,
                window=self.window, q_norm_w=qw, k_norm_w=kw, norm_eps=cfg.rms_norm_eps, norm_offset=cfg.norm_weight_offset)
        if x.is_cuda and x.shape[0] <= 128 and self.qkv.q_mult == 1 and _FUSE_QKV_DECODE:
            # decode-sized: the projection leaves its split-K partials and one kernel folds them, adds the
            # bias, normalises q / k heads, rotates and appends to the cache
            part = gemm.gemm_partials(coll.copy_to_tp(x), self.qkv.weight)
            if isinstance(part, gemm.SplitKPartial):
                kc, vc, ks, vs = self.kv_cache
                qkv = pa.fold_rope_append_kv(
                    part, self.qkv.bias, positions, meta.slot_mapping, kc, vc, ks, vs, self.hq, self.hkv, self.d,
                    theta=cfg.rope_theta, rot_dim=self.rot_dim, inv_freq=self.inv_freq, interleaved=self.rope_interleaved,
                    q_norm_w=qw, k_norm_w=kw, norm_eps=cfg.rms_norm_eps, norm_offset=cfg.norm_weight_offset)
                return self._attend_cached(qkv, meta)
            qkv = part if self.qkv.bias is None else part + self.qkv.bias
        else:
            qkv = self.qkv(x)
        return self._infer(qkv, positions, meta, qw, kw)

    def _infer(self, qkv, positions, meta: InferMeta, qw, kw):
        cfg = self.cfg
        hq, hkv, d = self.hq, self.hkv, self.d
        if qw is not None:
            q3 = qkv[:, : hq * d].unflatten(1, (hq, d))
            k3 = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
            if qkv.is_cuda:
                attn_ops._headnorm_fwd(q3, qw, cfg.norm_weight_offset, q3, cfg.rms_norm_eps)
                attn_ops._headnorm_fwd(k3, kw, cfg.norm_weight_offset, k3, cfg.rms_norm_eps)
            else:
                q3.copy_(attn_ops._headnorm_reference(q3, qw, cfg.rms_norm_eps, cfg.norm_weight_offset))
                k3.copy_(attn_ops._headnorm_reference(k3, kw, cfg.rms_norm_eps, cfg.norm_weight_offset))
        kc, vc, ks, vs = self.kv_cache
        pa.rope_append_kv(qkv, positions, meta.slot_mapping, kc, vc, ks, vs, hq, hkv, d, theta=cfg.rope_theta,
                          rot_dim=self.rot_dim, inv_freq=self.inv_freq, interleaved=self.rope_interleaved)
        return self._attend_cached(qkv, meta)

    def _attend_cached(self, qkv, meta: InferMeta):
        """Attention over the paged cache for a ``qkv`` whose q / k are rotated and whose k / v are appended."""
        hq, hkv, d = self.hq, self.hkv, self.d
        t = qkv.shape[0]
        kc, vc, ks, vs = self.kv_cache
        q = qkv[:, : hq * d].unflatten(1, (hq, d))
        if meta.mode == "decode":
            out = pa.paged_decode(q, kc, vc, ks, vs, meta.block_table, meta.seq_lens, self.scale,
                                  max_context=meta.max_context, window=self.window)
            return out.view(t, hq * d)
        k = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
        v = qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, d))
        if meta.has_history:
            k, v = _gather_history(self.kv_cache, meta, hkv, d)
        o, _ = attn_ops.attention_forward(q, k, v, meta.varlen, self.scale, True, self.window, need_lse=False)
        return o.view(t, hq * d)


def _gather_history(kv_cache, meta: InferMeta, hkv: int, d: int):
    """Contiguous K/V (cached prefix + the chunk just appended) for every sequence of a prefill
    chunk, read back from the paged cache; used only when a prompt spans several chunks."""
    kc, vc, ks, vs = kv_cache
    slots = meta.history  # int64 [total_k] cache slots in packed key order
    pages, offs = slots // pa.PAGE, slots % pa.PAGE
    if kc.dtype == torch.uint8:
        k = (kc.view(torch.float8_e4m3fn)[pages, :, offs].float() * ks[pages, :, offs].unsqueeze(-1)).to(torch.bfloat16)
        v = (vc.view(torch.float8_e4m3fn)[pages, :, offs].float() * vs[pages, :, offs].unsqueeze(-1)).to(torch.bfloat16)
    else:
        k, v = kc[pages, :, offs], vc[pages, :, offs]
    return k.contiguous(), v.contiguous()


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device, mlp: nn.Module | None = None,
                 attn: nn.Module | None = None):
        super().__init__()
        self.input_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, cfg.norm_weight_offset)
        self.attn = attn if attn is not None else Attention(cfg, layer_idx, dtype, device)
        self.post_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, cfg.norm_weight_offset)
        self.mlp = mlp if mlp is not None else GatedMLP(cfg.hidden_size, cfg.intermediate_size, cfg.hidden_act,
                                                        cfg.use_bias, dtype, device)
        # both row-parallel outputs of this block feed an RMSNorm with residual
        out_proj = getattr(self.attn, "o", None) or getattr(self.attn, "out_proj", None)
        if out_proj is not None:
            out_proj.defer_reduce = True
        if isinstance(self.mlp, GatedMLP):
            self.mlp.down.defer_reduce = True

    def forward(self, x, residual, positions, meta):
        sp = isinstance(meta, TrainMeta) and meta.sequence_parallel
        # the region is opened here, not by the caller, so that a recompute under activation checkpointing sees it too
        with coll.sequence_parallel_region(sp):
            sp = coll.in_sequence_parallel()
            if residual is None and isinstance(x, TpPartial):
                # the embedding lookup is still spread over the TP group: its sum is the residual stream
                h, residual = self.input_norm(x, None, want_sum=True)
            elif residual is None:
                residual = x
                h = self.input_norm(x)
            else:
                h, residual = self.input_norm(x, residual)
            if sp:
                h = coll.gather_rows(h)          # [T / tp, H] -> [T, H]; backward reduce-scatters the input gradient
            h = self.attn(h, positions, meta)    # row-parallel output: reduce-scattered back to [T / tp, H] when sp
            h, residual = self.post_norm(h, residual)
            if sp:
                h = coll.gather_rows(h)
            h = self.mlp(h)
        return h, residual


def _layer_done(hook, li: int):
    def fire(_grad):
        hook(li)   # the gradient itself is left untouched
    return fire


class DenseCausalLM(nn.Module):
    """Embedding -> N x DecoderLayer -> final norm; ``lm_head`` is applied by the caller."""

    supports_sequence_parallel = True     # subclasses with their own forward loop switch this off

    def __init__(self, cfg: ModelConfig, device="cpu", dtype: torch.dtype | None = None):
        super().__init__()
        dtype = dtype or cfg.dtype
        self.cfg = cfg
        self.embed = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device, cfg.embed_scale)
        self.layers = nn.ModuleList([self._make_layer(i, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, cfg.norm_weight_offset)
        self.lm_head = VocabParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device,
                                           tied_to=self.embed if cfg.tie_word_embeddings else None)
        self._kv_spec = None
        # layer 0 starts with ``input_norm`` of the embedding output, so that norm can take the embedding lookup
        # un-reduced; only claimed for the stock layer / model forward (families with their own are left alone)
        self._first_norm_takes_partial = (type(self.layers[0]).forward is DecoderLayer.forward
                                          and type(self).forward is DenseCausalLM.forward)

    def _make_layer(self, i, dtype, device):
        return DecoderLayer(self.cfg, i, dtype, device)

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids, position_ids, meta) -> CausalLMOutput:
        ids = input_ids.reshape(-1)
        positions = position_ids.reshape(-1)
        if positions.dtype != torch.int32:
            positions = positions.to(torch.int32)
        sp = (isinstance(meta, TrainMeta) and meta.sequence_parallel and self.supports_sequence_parallel
              and get_context().tp_size > 1)
        tokens = ids.numel()
        if isinstance(meta, TrainMeta) and meta.sequence_parallel != sp:
            meta = dataclasses.replace(meta, sequence_parallel=sp)
        if sp:
            # rows are dealt out in equal shares: pad the packed batch with one throw-away sequence
            pad = (-tokens) % get_context().tp_size
            if pad:
                ids = torch.cat([ids, ids.new_zeros(pad)])
                positions = torch.cat([positions, torch.arange(pad, dtype=positions.dtype, device=positions.device)])
                host = meta.varlen.cu_q_host
                lens = [b - a for a, b in zip(host[:-1], host[1:])] + [pad]
                meta = dataclasses.replace(meta, varlen=attn_ops.build_varlen_meta(lens, device=ids.device))
            with coll.sequence_parallel_region(True):
                x = self.embed(ids)            # the vocabulary-parallel sum becomes a reduce-scatter: [T / tp, H]
        else:
            # inference with a peer-memory communicator: the first norm folds the vocabulary-parallel sum in
            x = self.embed(ids, defer_reduce=isinstance(meta, InferMeta) and self._first_norm_takes_partial)
        residual = None
        use_ckpt = isinstance(meta, TrainMeta) and meta.activation_checkpointing and torch.is_grad_enabled()
        n_ckpt = len(self.layers)
        if use_ckpt and meta.checkpoint_layers is not None:
            n_ckpt = max(0, min(n_ckpt, int(meta.checkpoint_layers)))
        grad_hook = meta.layer_grad_hook if isinstance(meta, TrainMeta) and torch.is_grad_enabled() else None
        for li, layer in enumerate(self.layers):
            if grad_hook is not None and x.requires_grad:
                x.register_hook(_layer_done(grad_hook, li))
            if use_ckpt and li < n_ckpt:
                if residual is None:
                    x, residual = checkpoint(_run_first, layer, x, positions, meta, use_reentrant=False)
                else:
                    x, residual = checkpoint(layer, x, residual, positions, meta, use_reentrant=False)
            else:
                x, residual = layer(x, residual, positions, meta)
        h, _ = self.norm(x, residual)
        if sp:
            # every rank needs all rows for the loss; the log-prob op hands back the complete gradient on every rank
            h = coll.gather_rows_same_grad(h)[:tokens]
        out = CausalLMOutput(hidden_states=h)
        if isinstance(meta, InferMeta):
            rows = h if meta.logit_rows is None else h.index_select(0, meta.logit_rows)
            out.logits_shard = self.compute_logits(rows, out_dtype=torch.float32)
        return out

    def compute_logits(self, hidden, out_dtype=torch.bfloat16):
        logits = self.lm_head(hidden, out_dtype=out_dtype)
        cap = self.cfg.final_logit_softcapping
        if cap:
            logits = (torch.tanh(logits.float() / cap) * cap).to(logits.dtype)
        return logits

    # --------------------------------------------------------- engine lifecycle
    def kv_cache_bytes_per_page(self, fp8: bool) -> int:
        hkv = self.layers[0].attn.hkv
        d = self.cfg.head_dim
        per = hkv * pa.PAGE * d * (1 if fp8 else 2) * 2
        if fp8:
            per += hkv * pa.PAGE * 4 * 2
        return per * len(self.layers)

    def allocate_kv_caches(self, num_pages: int, fp8: bool = False) -> None:
        dev = self.embed.weight.device
        for layer in self.layers:
            a = layer.attn
            a.kv_cache = pa.alloc_kv_cache(num_pages, a.hkv, a.d, dev, fp8)
        self._kv_spec = (num_pages, fp8)

    def set_kv_caches(self, caches) -> None:
        for layer, c in zip(self.layers, caches):
            layer.attn.kv_cache = c

    def kv_caches(self):
        return [layer.attn.kv_cache for layer in self.layers]

    def clear_kv_caches(self) -> None:
        for layer in self.layers:
            layer.attn.kv_cache = None
        self._kv_spec = None

    def reset_kv_caches(self) -> None:
        """Nothing to zero: pages are only read below ``seq_lens``."""

    def offload_train_weights(self) -> None:
        for p in self.parameters():
            p.data = p.data.to("cpu", non_blocking=True)

    def onload_train_weights(self, device) -> None:
        for p in self.parameters():
            p.data = p.data.to(device, non_blocking=True)

    def finalize_router_expert_bias(self, tp_group=None, dp_group=None) -> None:
        pass


def _run_first(layer, x, positions, meta):
    return layer(x, None, positions, meta)


def init_weights(model: nn.Module, seed: int = 0, std: float = 0.02) -> None:
    """Seeded random init (normal(0, std) for matrices, ones for norm scales, zeros for biases)."""
    gen_cpu = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            rng = getattr(p, "expert_range", None)
            if rng is not None:
                # stacked expert weights: expert e gets the same values whichever rank holds it (expert-parallel,
                # TP-sharded or all on one device), from a generator seeded by the parameter name and e
                base = seed + (zlib.crc32(name.encode()) % 100003)
                for le in range(p.shape[0]):
                    g = torch.Generator(device=p.device if p.is_cuda else "cpu").manual_seed(base + 7919 * (rng[0] + le + 1))
                    if p.is_cuda:
                        p[le].normal_(0.0, std, generator=g)
                    else:
                        p[le].copy_(torch.randn(p.shape[1:], generator=g) * std)
                continue
            if p.dim() >= 2:
                if p.is_cuda:
                    g = torch.Generator(device=p.device).manual_seed(seed + (zlib.crc32(name.encode()) % 100003))
                    p.normal_(0.0, std, generator=g)
                else:
                    p.copy_(torch.randn(p.shape, generator=gen_cpu) * std)
            elif "norm" in name:
                p.fill_(1.0 if getattr(model, "cfg", None) is None or model.cfg.norm_weight_offset == 0.0 else 0.0)
            else:
                p.zero_()
