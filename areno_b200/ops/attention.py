"""Variable-length causal attention (training and prefill) with GQA.

``VarlenMeta`` carries the per-batch sequence boundaries in the forms the kernels need (device
``cu_seqlens`` plus a per-sequence prefix of 64-row tiles for the CTA → (sequence, tile) map);
it is built once per packed batch on the host and shared by every layer.

``qkv_attention`` is the training entry point: it takes the fused QKV projection output,
applies RoPE in place, runs the flash-style forward, and in the backward writes dQ/dK/dV
straight into one packed buffer that is the gradient of the QKV projection.

Replaces ``flash_attn_varlen_func`` / SDPA usage in the reference
(``areno/engine/layers/attention_backend/train.py:126-257``); the fp32 restatement below
plays the role of its ``native`` backend as a consistency oracle.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from .rope import _rope_inplace, rope_reference

TILE = 64


@dataclass
class VarlenMeta:
    cu_q: torch.Tensor          # int32 [num_seqs + 1] on device
    cu_k: torch.Tensor          # int32 [num_seqs + 1] on device
    tile_prefix_q: torch.Tensor  # int32 [num_seqs + 1] on device
    tile_prefix_k: torch.Tensor  # int32 [num_seqs + 1] on device
    num_seqs: int
    total_q: int
    total_k: int
    total_q_tiles: int
    total_k_tiles: int
    max_q: int
    max_k: int
    cu_q_host: list[int]
    cu_k_host: list[int]


def build_varlen_meta(q_lens, k_lens=None, device="cpu") -> VarlenMeta:
    """q_lens / k_lens: python ints per sequence (k_lens defaults to q_lens)."""
    q_lens = [int(x) for x in q_lens]
    k_lens = q_lens if k_lens is None else [int(x) for x in k_lens]
    cu_q, cu_k, tq, tk = [0], [0], [0], [0]
    for lq, lk in zip(q_lens, k_lens):
        cu_q.append(cu_q[-1] + lq)
        cu_k.append(cu_k[-1] + lk)
        tq.append(tq[-1] + (lq + TILE - 1) // TILE)
        tk.append(tk[-1] + (lk + TILE - 1) // TILE)
    packed = torch.tensor([cu_q, cu_k, tq, tk], dtype=torch.int32)
    if str(device) != "cpu":
        packed = packed.pin_memory().to(device, non_blocking=True) if torch.cuda.is_available() else packed
    return VarlenMeta(
        cu_q=packed[0], cu_k=packed[1], tile_prefix_q=packed[2], tile_prefix_k=packed[3],
        num_seqs=len(q_lens), total_q=cu_q[-1], total_k=cu_k[-1], total_q_tiles=tq[-1], total_k_tiles=tk[-1],
        max_q=max(q_lens) if q_lens else 0, max_k=max(k_lens) if k_lens else 0, cu_q_host=cu_q, cu_k_host=cu_k,
    )


def attention_reference(q, k, v, meta: VarlenMeta, scale, causal=True, window=0):
    """fp32 oracle.  q: [Tq, Hq, D]; k, v: [Tk, Hkv, D] -> ([Tq, Hq, D], lse [Hq, Tq])."""
    hq, hkv = q.shape[1], k.shape[1]
    group = hq // hkv
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    lse = torch.zeros((hq, q.shape[0]), dtype=torch.float32, device=q.device)
    for s in range(meta.num_seqs):
        q0, q1 = meta.cu_q_host[s], meta.cu_q_host[s + 1]
        k0, k1 = meta.cu_k_host[s], meta.cu_k_host[s + 1]
        lq, lk = q1 - q0, k1 - k0
        if lq == 0:
            continue
        qs = q[q0:q1].float().transpose(0, 1)                                   # [Hq, lq, D]
        ks = k[k0:k1].float().transpose(0, 1).repeat_interleave(group, dim=0)   # [Hq, lk, D]
        vs = v[k0:k1].float().transpose(0, 1).repeat_interleave(group, dim=0)
        sc = torch.matmul(qs, ks.transpose(1, 2)) * scale
        i = torch.arange(lq, device=q.device)[:, None]
        j = torch.arange(lk, device=q.device)[None, :]
        mask = torch.ones((lq, lk), dtype=torch.bool, device=q.device)
        if causal:
            mask &= j <= i + (lk - lq)
        if window and window > 0:
            mask &= j > i + (lk - lq) - window
        sc = sc.masked_fill(~mask, float("-inf"))
        l = torch.logsumexp(sc, dim=-1)
        p = torch.exp(sc - l.unsqueeze(-1))
        out[q0:q1] = torch.matmul(p, vs).transpose(0, 1)
        lse[:, q0:q1] = l
    return out.to(q.dtype), lse


def _heads_view(t2d, col0, heads, d):
    return t2d[:, col0:col0 + heads * d].unflatten(1, (heads, d))


def attention_forward(q, k, v, meta: VarlenMeta, scale, causal=True, window=0, out=None, need_lse=True):
    """Kernel forward on [T, H, D] views (unit stride on D, head stride D, any token stride)."""
    if not q.is_cuda:
        o, lse = attention_reference(q, k, v, meta, scale, causal, window)
        return o, lse
    tq, hq, d = q.shape
    hkv = k.shape[1]
    for t in (q, k, v):
        assert t.dtype == torch.bfloat16 and t.stride(2) == 1 and t.stride(1) == d
    if out is None:
        out = torch.empty((tq, hq, d), dtype=q.dtype, device=q.device)
    lse = torch.empty((hq, tq), dtype=torch.float32, device=q.device) if need_lse else None
    _lib.call(
        "areno_attn_fwd",
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _lib.ptr(lse),
        meta.cu_q.data_ptr(), meta.cu_k.data_ptr(), meta.tile_prefix_q.data_ptr(),
        meta.num_seqs, meta.total_q_tiles, hq, hkv, d,
        q.stride(0), k.stride(0), v.stride(0), out.stride(0),
        float(scale), int(causal), int(window or 0), _lib.stream(),
    )
    return out, lse


def attention_backward(q, k, v, o, do, lse, meta: VarlenMeta, scale, causal, window, dq, dk, dv):
    tq, hq, d = q.shape
    hkv = k.shape[1]
    if do.stride(2) != 1 or do.stride(1) != d:
        do = do.contiguous()
    delta = torch.empty((hq, tq), dtype=torch.float32, device=q.device)
    _lib.call(
        "areno_attn_bwd",
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
        meta.cu_q.data_ptr(), meta.cu_k.data_ptr(), meta.tile_prefix_q.data_ptr(), meta.tile_prefix_k.data_ptr(),
        meta.num_seqs, meta.total_q_tiles, meta.total_k_tiles, meta.total_q, hq, hkv, d,
        q.stride(0), k.stride(0), v.stride(0), o.stride(0), do.stride(0), dq.stride(0), dk.stride(0), dv.stride(0),
        float(scale), int(causal), int(window or 0), _lib.stream(),
    )


class _VarlenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta, scale, causal, window):
        o, lse = attention_forward(q, k, v, meta, scale, causal, window)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta, ctx.args = meta, (scale, causal, window)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, window = ctx.args
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        attention_backward(q, k, v, o, do, lse, ctx.meta, scale, causal, window, dq, dk, dv)
        return dq, dk, dv, None, None, None, None


def varlen_attention(q, k, v, meta: VarlenMeta, scale: float, causal: bool = True, window: int = 0):
    """Differentiable attention on separate q/k/v tensors ([T, H, D], contiguous)."""
    if not q.is_cuda:
        return _reference_autograd(q, k, v, meta, scale, causal, window)
    q, k, v = (t if (t.stride(2) == 1 and t.stride(1) == t.shape[2]) else t.contiguous() for t in (q, k, v))
    return _VarlenAttention.apply(q, k, v, meta, scale, causal, window)


def _reference_autograd(q, k, v, meta, scale, causal, window):
    # differentiable fp32 path for CPU tensors
    hq, hkv = q.shape[1], k.shape[1]
    group = hq // hkv
    outs = []
    for s in range(meta.num_seqs):
        q0, q1 = meta.cu_q_host[s], meta.cu_q_host[s + 1]
        k0, k1 = meta.cu_k_host[s], meta.cu_k_host[s + 1]
        lq, lk = q1 - q0, k1 - k0
        qs = q[q0:q1].float().transpose(0, 1)
        ks = k[k0:k1].float().transpose(0, 1).repeat_interleave(group, dim=0)
        vs = v[k0:k1].float().transpose(0, 1).repeat_interleave(group, dim=0)
        sc = torch.matmul(qs, ks.transpose(1, 2)) * scale
        i = torch.arange(lq, device=q.device)[:, None]
        j = torch.arange(lk, device=q.device)[None, :]
        mask = torch.ones((lq, lk), dtype=torch.bool, device=q.device)
        if causal:
            mask &= j <= i + (lk - lq)
        if window and window > 0:
            mask &= j > i + (lk - lq) - window
        sc = sc.masked_fill(~mask, float("-inf"))
        outs.append(torch.matmul(torch.softmax(sc, dim=-1), vs).transpose(0, 1))
    return torch.cat(outs, dim=0).to(q.dtype)


class _QKVAttention(torch.autograd.Function):
    """Fused RoPE + attention on the packed QKV projection output ``[T, (Hq + 2 Hkv) D]``."""

    @staticmethod
    def forward(ctx, qkv, positions, meta, hq, hkv, d, scale, theta, rot_dim, inv_freq, interleaved, causal,
                window):
        assert qkv.is_contiguous()
        q = _heads_view(qkv, 0, hq, d)
        k = _heads_view(qkv, hq * d, hkv, d)
        v = _heads_view(qkv, (hq + hkv) * d, hkv, d)
        if rot_dim > 0:
            _rope_inplace(q, positions, theta, rot_dim, inv_freq, interleaved, 1.0)
            _rope_inplace(k, positions, theta, rot_dim, inv_freq, interleaved, 1.0)
        o, lse = attention_forward(q, k, v, meta, scale, causal, window)
        ctx.save_for_backward(qkv, o, lse, positions, *([inv_freq] if inv_freq is not None else []))
        ctx.meta = meta
        ctx.args = (hq, hkv, d, scale, theta, rot_dim, interleaved, causal, window, inv_freq is not None)
        return o.view(o.shape[0], hq * d)

    @staticmethod
    def backward(ctx, do):
        saved = ctx.saved_tensors
        qkv, o, lse, positions = saved[:4]
        hq, hkv, d, scale, theta, rot_dim, interleaved, causal, window, has_freq = ctx.args
        inv_freq = saved[4] if has_freq else None
        q = _heads_view(qkv, 0, hq, d)
        k = _heads_view(qkv, hq * d, hkv, d)
        v = _heads_view(qkv, (hq + hkv) * d, hkv, d)
        dqkv = torch.empty_like(qkv)
        dq = _heads_view(dqkv, 0, hq, d)
        dk = _heads_view(dqkv, hq * d, hkv, d)
        dv = _heads_view(dqkv, (hq + hkv) * d, hkv, d)
        do3 = do.reshape(do.shape[0], hq, d)
        attention_backward(q, k, v, o, do3, lse, ctx.meta, scale, causal, window, dq, dk, dv)
        if rot_dim > 0:
            _rope_inplace(dq, positions, theta, rot_dim, inv_freq, interleaved, -1.0)
            _rope_inplace(dk, positions, theta, rot_dim, inv_freq, interleaved, -1.0)
        return (dqkv,) + (None,) * 12


def qkv_attention(qkv, positions, meta: VarlenMeta, hq: int, hkv: int, d: int, scale: float | None = None,
                  theta: float = 10000.0, rot_dim: int | None = None, inv_freq=None, interleaved: bool = False,
                  causal: bool = True, window: int = 0):
    """RoPE + causal attention on a packed ``[T, (Hq + 2 Hkv) D]`` projection output.

    On CUDA, ``qkv`` is rotated in place (it is the private output of the QKV GEMM).
    Returns ``[T, Hq D]``.
    """
    scale = d ** -0.5 if scale is None else scale
    rot = d if rot_dim is None else rot_dim
    if not qkv.is_cuda:
        t = qkv.shape[0]
        q = qkv[:, : hq * d].reshape(t, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].reshape(t, hkv, d)
        v = qkv[:, (hq + hkv) * d:].reshape(t, hkv, d)
        if rot > 0:
            q = _rope_diff(q, positions, theta, rot, inv_freq, interleaved)
            k = _rope_diff(k, positions, theta, rot, inv_freq, interleaved)
        return _reference_autograd(q, k, v, meta, scale, causal, window).reshape(t, hq * d)
    if positions.dtype != torch.int32:
        positions = positions.to(torch.int32)
    return _QKVAttention.apply(qkv, positions, meta, hq, hkv, d, scale, theta, rot, inv_freq, interleaved, causal,
                               window)


def _rope_diff(x, positions, theta, rot, inv_freq, interleaved):
    """Differentiable RoPE for the CPU path (no in-place writes)."""
    half = rot // 2
    if inv_freq is None:
        inv_freq = theta ** (-torch.arange(0, half, dtype=torch.float32, device=x.device) * 2.0 / rot)
    ang = positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0:rot:2], xf[..., 1:rot:2]
        ra, rb = a * cos - b * sin, b * cos + a * sin
        rotated = torch.stack([ra, rb], dim=-1).flatten(-2)
    else:
        a, b = xf[..., :half], xf[..., half:rot]
        rotated = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    return torch.cat([rotated, xf[..., rot:]], dim=-1).to(x.dtype)


__all__ = [
    "VarlenMeta", "build_varlen_meta", "attention_reference", "attention_forward", "attention_backward",
    "varlen_attention", "qkv_attention", "rope_reference",
]
