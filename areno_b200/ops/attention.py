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

import os

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
    tile_prefix_q128: torch.Tensor | None = None   # int32 [num_seqs + 1]: 128-row query tiles (tcgen05 forward)
    total_q_tiles128: int = 0


def build_varlen_meta(q_lens, k_lens=None, device="cpu") -> VarlenMeta:
    """q_lens / k_lens: python ints per sequence (k_lens defaults to q_lens)."""
    q_lens = [int(x) for x in q_lens]
    k_lens = q_lens if k_lens is None else [int(x) for x in k_lens]
    cu_q, cu_k, tq, tk, tq128 = [0], [0], [0], [0], [0]
    for lq, lk in zip(q_lens, k_lens):
        cu_q.append(cu_q[-1] + lq)
        cu_k.append(cu_k[-1] + lk)
        tq.append(tq[-1] + (lq + TILE - 1) // TILE)
        tk.append(tk[-1] + (lk + TILE - 1) // TILE)
        tq128.append(tq128[-1] + (lq + 127) // 128)
    packed = torch.tensor([cu_q, cu_k, tq, tk, tq128], dtype=torch.int32)
    if str(device) != "cpu":
        packed = packed.pin_memory().to(device, non_blocking=True) if torch.cuda.is_available() else packed
    return VarlenMeta(
        cu_q=packed[0], cu_k=packed[1], tile_prefix_q=packed[2], tile_prefix_k=packed[3],
        num_seqs=len(q_lens), total_q=cu_q[-1], total_k=cu_k[-1], total_q_tiles=tq[-1], total_k_tiles=tk[-1],
        max_q=max(q_lens) if q_lens else 0, max_k=max(k_lens) if k_lens else 0, cu_q_host=cu_q, cu_k_host=cu_k,
        tile_prefix_q128=packed[4], total_q_tiles128=tq128[-1],
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


# ARENO_ATTN_TC=0 keeps the mma.sync forward for head size 128 as well (A/B timing).
_TC_FORWARD = os.environ.get("ARENO_ATTN_TC", "1") != "0"


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
    if d in (64, 128) and not window and _TC_FORWARD and meta.tile_prefix_q128 is not None:
        # tcgen05 / TMEM kernel: 128 x 128 tiles, TMA-fed, softmax between the two MMAs
        _lib.call(
            "areno_attn_fwd_tc",
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _lib.ptr(lse),
            meta.cu_q.data_ptr(), meta.cu_k.data_ptr(), meta.tile_prefix_q128.data_ptr(),
            meta.num_seqs, meta.total_q_tiles128, hq, hkv, d, tq, k.shape[0],
            q.stride(0), k.stride(0), v.stride(0), out.stride(0),
            float(scale), int(causal), _lib.status_buffer(q.device).data_ptr(), _lib.stream(),
        )
        return out, lse
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
    # grouped-query attention: dK / dV are computed per query head (seven times the CTAs at 28 / 4 heads, no
    # CTA that loops over the whole group) and summed over the group from this fp32 scratch
    tk, group = k.shape[0], hq // hkv
    ws = torch.empty((2, group, tk, hkv * d), dtype=torch.float32, device=q.device) if group > 1 else None
    _lib.call(
        "areno_attn_bwd",
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
        meta.cu_q.data_ptr(), meta.cu_k.data_ptr(), meta.tile_prefix_q.data_ptr(), meta.tile_prefix_k.data_ptr(),
        meta.num_seqs, meta.total_q_tiles, meta.total_k_tiles, meta.total_q, hq, hkv, d,
        q.stride(0), k.stride(0), v.stride(0), o.stride(0), do.stride(0), dq.stride(0), dk.stride(0), dv.stride(0),
        float(scale), int(causal), int(window or 0), ws.data_ptr() if ws is not None else None, tk, _lib.stream(),
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


def _headnorm_fwd(x3, w, w_offset, y3, eps):
    """x3, y3: [T, heads, D] strided views; returns inv_rms [T * heads]."""
    t, heads, d = x3.shape
    inv = torch.empty(t * heads, dtype=torch.float32, device=x3.device)
    _lib.call("areno_headnorm_fwd", x3.data_ptr(), x3.stride(0), w.data_ptr(), int(w.dtype == torch.float32),
              float(w_offset), y3.data_ptr(), y3.stride(0), inv.data_ptr(), t, heads, d, float(eps), _lib.stream())
    return inv


def _headnorm_bwd(dy3, x3, w, w_offset, inv, dx3):
    """Returns fp32 dW [D] (or None when accumulated into ``w.main_grad``)."""
    t, heads, d = x3.shape
    nblk = _lib.fn("areno_headnorm_bwd_blocks")(t * heads)
    partial = torch.empty((nblk, d), dtype=torch.float32, device=x3.device)
    main_grad = getattr(w, "main_grad", None)
    if main_grad is not None:
        target, acc = main_grad, 1
        w.grad_added_to_main_grad = True
    else:
        target, acc = torch.empty(d, dtype=torch.float32, device=x3.device), 0
    _lib.call("areno_headnorm_bwd", dy3.data_ptr(), dy3.stride(0), x3.data_ptr(), x3.stride(0), w.data_ptr(),
              int(w.dtype == torch.float32), float(w_offset), inv.data_ptr(), dx3.data_ptr(), dx3.stride(0),
              partial.data_ptr(), target.data_ptr(), acc, t, heads, d, _lib.stream())
    return None if acc else target.to(w.dtype)


class _QKVAttention(torch.autograd.Function):
    """Fused (q/k head-norm +) RoPE + attention on the packed QKV projection output
    ``[T, (Hq + 2 Hkv) D]``."""

    @staticmethod
    def forward(ctx, qkv, q_norm_w, k_norm_w, positions, meta, hq, hkv, d, scale, theta, rot_dim, inv_freq,
                interleaved, causal, window, norm_eps, norm_offset):
        assert qkv.is_contiguous()
        q = _heads_view(qkv, 0, hq, d)
        k = _heads_view(qkv, hq * d, hkv, d)
        v = _heads_view(qkv, (hq + hkv) * d, hkv, d)
        has_norm = q_norm_w is not None
        inv_q = inv_k = qk2 = None
        if has_norm:
            qk2 = torch.empty((qkv.shape[0], (hq + hkv) * d), dtype=qkv.dtype, device=qkv.device)
            qn = _heads_view(qk2, 0, hq, d)
            kn = _heads_view(qk2, hq * d, hkv, d)
            inv_q = _headnorm_fwd(q, q_norm_w, norm_offset, qn, norm_eps)
            inv_k = _headnorm_fwd(k, k_norm_w, norm_offset, kn, norm_eps)
            q, k = qn, kn
        if rot_dim > 0:
            # q heads are followed directly by k heads in both buffers: one launch rotates both
            qk = _heads_view(qk2 if has_norm else qkv, 0, hq + hkv, d)
            _rope_inplace(qk, positions, theta, rot_dim, inv_freq, interleaved, 1.0)
        o, lse = attention_forward(q, k, v, meta, scale, causal, window)
        extras = []
        if inv_freq is not None:
            extras.append(inv_freq)
        if has_norm:
            extras += [qk2, inv_q, inv_k, q_norm_w, k_norm_w]
        ctx.save_for_backward(qkv, o, lse, positions, *extras)
        ctx.meta = meta
        ctx.args = (hq, hkv, d, scale, theta, rot_dim, interleaved, causal, window, inv_freq is not None, has_norm,
                    norm_offset)
        return o.view(o.shape[0], hq * d)

    @staticmethod
    def backward(ctx, do):
        saved = list(ctx.saved_tensors)
        qkv, o, lse, positions = saved[:4]
        rest = saved[4:]
        hq, hkv, d, scale, theta, rot_dim, interleaved, causal, window, has_freq, has_norm, norm_offset = ctx.args
        inv_freq = rest.pop(0) if has_freq else None
        v = _heads_view(qkv, (hq + hkv) * d, hkv, d)
        dqkv = torch.empty_like(qkv)
        dv = _heads_view(dqkv, (hq + hkv) * d, hkv, d)
        do3 = do.reshape(do.shape[0], hq, d)
        dwq = dwk = None
        if has_norm:
            qk2, inv_q, inv_k, q_norm_w, k_norm_w = rest
            q = _heads_view(qk2, 0, hq, d)
            k = _heads_view(qk2, hq * d, hkv, d)
            dqk2 = torch.empty_like(qk2)
            dq = _heads_view(dqk2, 0, hq, d)
            dk = _heads_view(dqk2, hq * d, hkv, d)
        else:
            q = _heads_view(qkv, 0, hq, d)
            k = _heads_view(qkv, hq * d, hkv, d)
            dq = _heads_view(dqkv, 0, hq, d)
            dk = _heads_view(dqkv, hq * d, hkv, d)
        attention_backward(q, k, v, o, do3, lse, ctx.meta, scale, causal, window, dq, dk, dv)
        if rot_dim > 0:
            dqk = _heads_view(dqk2 if has_norm else dqkv, 0, hq + hkv, d)
            _rope_inplace(dqk, positions, theta, rot_dim, inv_freq, interleaved, -1.0)
        if has_norm:
            dwq = _headnorm_bwd(dq, _heads_view(qkv, 0, hq, d), q_norm_w, norm_offset, inv_q,
                                _heads_view(dqkv, 0, hq, d))
            dwk = _headnorm_bwd(dk, _heads_view(qkv, hq * d, hkv, d), k_norm_w, norm_offset, inv_k,
                                _heads_view(dqkv, hq * d, hkv, d))
        return (dqkv, dwq, dwk) + (None,) * 14


class _HeadRmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x3, w, offset, eps):
        y3 = torch.empty_like(x3)
        inv = _headnorm_fwd(x3, w, offset, y3, eps)
        ctx.save_for_backward(x3, w, inv)
        ctx.offset = offset
        return y3

    @staticmethod
    def backward(ctx, dy):
        x3, w, inv = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x3)
        dw = _headnorm_bwd(dy, x3, w, ctx.offset, inv, dx)
        return dx, (dw if ctx.needs_input_grad[1] else None), None, None


def head_rmsnorm(x3, w, eps: float = 1e-6, offset: float = 0.0):
    """RMSNorm over the last dim of ``[T, heads, D]`` (per-head q / k / v norms).  ``w=None`` normalises
    without a learned scale."""
    if w is None:
        w = torch.ones(x3.shape[-1], dtype=torch.float32, device=x3.device)
    if not x3.is_cuda:
        return _headnorm_reference(x3, w, eps, offset)
    x3 = x3.contiguous()
    return _HeadRmsNorm.apply(x3, w, float(offset), float(eps))


def _headnorm_reference(x, w, eps, offset):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + offset)
    return y.to(x.dtype)


def qkv_attention(qkv, positions, meta: VarlenMeta, hq: int, hkv: int, d: int, scale: float | None = None,
                  theta: float = 10000.0, rot_dim: int | None = None, inv_freq=None, interleaved: bool = False,
                  causal: bool = True, window: int = 0, q_norm_w=None, k_norm_w=None, norm_eps: float = 1e-6,
                  norm_offset: float = 0.0):
    """(per-head q/k RMSNorm +) RoPE + causal attention on a packed ``[T, (Hq + 2 Hkv) D]`` projection
    output.  On CUDA, ``qkv`` is rotated in place when no head norm is used (it is the private
    output of the QKV GEMM).  Returns ``[T, Hq D]``.
    """
    scale = d ** -0.5 if scale is None else scale
    rot = d if rot_dim is None else rot_dim
    if not qkv.is_cuda:
        t = qkv.shape[0]
        q = qkv[:, : hq * d].reshape(t, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].reshape(t, hkv, d)
        v = qkv[:, (hq + hkv) * d:].reshape(t, hkv, d)
        if q_norm_w is not None:
            q = _headnorm_reference(q, q_norm_w, norm_eps, norm_offset)
            k = _headnorm_reference(k, k_norm_w, norm_eps, norm_offset)
        if rot > 0:
            q = _rope_diff(q, positions, theta, rot, inv_freq, interleaved)
            k = _rope_diff(k, positions, theta, rot, inv_freq, interleaved)
        return _reference_autograd(q, k, v, meta, scale, causal, window).reshape(t, hq * d)
    if positions.dtype != torch.int32:
        positions = positions.to(torch.int32)
    return _QKVAttention.apply(qkv, q_norm_w, k_norm_w, positions, meta, hq, hkv, d, scale, theta, rot, inv_freq,
                               interleaved, causal, window, norm_eps, norm_offset)


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
