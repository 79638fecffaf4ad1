"""Rotary position embedding applied in place on packed ``[tokens, heads, head_dim]`` views.

Variants: full or partial rotation (``rot_dim < head_dim``), NeoX rotate-half or GPT-J
interleaved pairing, optional explicit ``inv_freq`` (scaled RoPE).  The backward is the
inverse rotation.  The reference does this with PyTorch ops traced by a compiler
(``areno/engine/layers/rotary.py:46-138``).
"""

from __future__ import annotations

import torch

from . import _lib


def rope_reference(x, positions, theta, rot_dim=None, inv_freq=None, interleaved=False, sign=1.0):
    """x: [tokens, heads, head_dim]; positions: [tokens]."""
    d = x.shape[-1]
    rot = d if rot_dim is None else rot_dim
    half = rot // 2
    if inv_freq is None:
        inv_freq = theta ** (-torch.arange(0, half, dtype=torch.float32, device=x.device) * 2.0 / rot)
    ang = positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = ang.cos()[:, None, :], (ang.sin() * sign)[:, None, :]
    xf = x.float()
    out = xf.clone()
    if interleaved:
        a, b = xf[..., 0:rot:2], xf[..., 1:rot:2]
        out[..., 0:rot:2] = a * cos - b * sin
        out[..., 1:rot:2] = b * cos + a * sin
    else:
        a, b = xf[..., :half], xf[..., half:rot]
        out[..., :half] = a * cos - b * sin
        out[..., half:rot] = b * cos + a * sin
    return out.to(x.dtype)


def _rope_inplace(x, positions, theta, rot_dim, inv_freq, interleaved, sign):
    # x: [tokens, heads, head_dim] view with unit stride on the last dim and head stride == head_dim
    tokens, heads, d = x.shape
    assert x.stride(2) == 1 and x.stride(1) == d
    _lib.call(
        "areno_rope", x.data_ptr(), positions.data_ptr(), _lib.ptr(inv_freq), tokens, heads, d, rot_dim,
        x.stride(0), float(theta), float(sign), int(interleaved), _lib.stream(),
    )


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, theta, rot_dim, inv_freq, interleaved):
        ctx.mark_dirty(x)
        _rope_inplace(x, positions, theta, rot_dim, inv_freq, interleaved, 1.0)
        ctx.save_for_backward(positions, inv_freq) if inv_freq is not None else ctx.save_for_backward(positions)
        ctx.has_freq = inv_freq is not None
        ctx.args = (theta, rot_dim, interleaved)
        return x

    @staticmethod
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        positions = saved[0]
        inv_freq = saved[1] if ctx.has_freq else None
        theta, rot_dim, interleaved = ctx.args
        dx = dy.clone() if not (dy.stride(2) == 1 and dy.stride(1) == dy.shape[2]) else dy.clone()
        _rope_inplace(dx, positions, theta, rot_dim, inv_freq, interleaved, -1.0)
        return dx, None, None, None, None, None


def apply_rope(x, positions, theta: float = 10000.0, rot_dim: int | None = None, inv_freq=None,
               interleaved: bool = False):
    """Rotate ``x`` ([tokens, heads, head_dim]).  On CUDA the rotation is done in place on ``x``
    (which must not be needed un-rotated afterwards) and ``x`` itself is returned."""
    rot = x.shape[-1] if rot_dim is None else rot_dim
    if not x.is_cuda:
        return rope_reference(x, positions, theta, rot, inv_freq, interleaved)
    if positions.dtype != torch.int32:
        positions = positions.to(torch.int32)
    if torch.is_grad_enabled() and x.requires_grad:
        return _Rope.apply(x, positions, theta, rot, inv_freq, interleaved)
    _rope_inplace(x, positions, theta, rot, inv_freq, interleaved, 1.0)
    return x
