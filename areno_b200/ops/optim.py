"""Fused optimizer steps on flat fp32 shards (AdamW fp32-master, AdamW with block-scaled 8-bit
moments), gradient sum-of-squares and scaling.  CPU tensors run an identical PyTorch restatement."""

from __future__ import annotations

import torch

from . import _lib

Q_BLOCK = 32


def adamw_fp32(master, m, v, grad, param_out, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
               scale_tensor=None):
    """One AdamW step on fp32 ``master``/``m``/``v`` given fp32 ``grad``; writes bf16 ``param_out``."""
    if not master.is_cuda:
        if scale_tensor is not None:
            grad_scale = grad_scale * float(scale_tensor[0])
        g = grad.float() * grad_scale
        if weight_decay != 0.0:
            master.mul_(1.0 - lr * weight_decay)
        m.mul_(beta1).add_(g, alpha=1.0 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
        bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        master.addcdiv_(m, v.sqrt().div_(bc2 ** 0.5).add_(eps), value=-lr / bc1)
        if param_out is not None:
            param_out.copy_(master)
        return
    _lib.call("areno_adamw_fp32", master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(),
              _lib.ptr(param_out), master.numel(), float(lr), float(beta1), float(beta2), float(eps),
              float(weight_decay), int(step), float(grad_scale), _lib.ptr(scale_tensor), _lib.stream())


def adamw_8bit(master, mq, vq, m_scale, v_scale, grad, param, lr, beta1, beta2, eps, weight_decay, step,
               grad_scale=1.0, scale_tensor=None):
    """AdamW with int8 ``mq`` / uint8 ``vq`` (sqrt of v) and one fp32 scale per 32 elements."""
    n = grad.numel()
    if not grad.is_cuda:
        if scale_tensor is not None:
            grad_scale = grad_scale * float(scale_tensor[0])
        nb = (n + Q_BLOCK - 1) // Q_BLOCK
        pad = nb * Q_BLOCK - n
        ms = m_scale.repeat_interleave(Q_BLOCK)[:n]
        vs = v_scale.repeat_interleave(Q_BLOCK)[:n]
        mf = mq.float() * ms
        sv = vq.float() * vs
        vf = sv * sv
        g = grad.float() * grad_scale
        mf = beta1 * mf + (1 - beta1) * g
        vf = beta2 * vf + (1 - beta2) * g * g
        src = master if master is not None else param
        p = src.float()
        bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        p = p * (1 - lr * weight_decay) - lr * (mf / bc1) / ((vf / bc2).sqrt() + eps)
        if master is not None:
            master.copy_(p)
        if param is not None:
            param.copy_(p.to(param.dtype))
        mp = torch.nn.functional.pad(mf, (0, pad)).view(nb, Q_BLOCK)
        sp = torch.nn.functional.pad(vf.sqrt(), (0, pad)).view(nb, Q_BLOCK)
        nms = mp.abs().amax(1).clamp_min(1e-30) / 127.0
        nvs = sp.amax(1).clamp_min(1e-30) / 255.0
        mq.copy_((mp / nms[:, None]).round().clamp(-127, 127).view(-1)[:n].to(torch.int8))
        vq.copy_((sp / nvs[:, None]).ceil().clamp(0, 255).view(-1)[:n].to(torch.uint8))
        m_scale.copy_(nms)
        v_scale.copy_(nvs)
        return
    _lib.call("areno_adamw_8bit", _lib.ptr(master), mq.data_ptr(), vq.data_ptr(), m_scale.data_ptr(),
              v_scale.data_ptr(), grad.data_ptr(), _lib.ptr(param), n, float(lr), float(beta1), float(beta2),
              float(eps), float(weight_decay), int(step), float(grad_scale), _lib.ptr(scale_tensor), _lib.stream())


_PARTIALS: dict[int, torch.Tensor] = {}


def sumsq(x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """Deterministic sum of squares of a flat fp32 tensor into a 1-element fp32 tensor."""
    if not x.is_cuda:
        val = x.float().pow(2).sum().reshape(1)
        if out is None:
            return val
        out.copy_(out + val if accumulate else val)
        return out
    assert x.dtype == torch.float32 and x.is_contiguous()
    idx = x.device.index
    part = _PARTIALS.get(idx)
    if part is None:
        part = torch.empty(_lib.fn("areno_sumsq_blocks")(), dtype=torch.float32, device=x.device)
        _PARTIALS[idx] = part
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    _lib.call("areno_sumsq", x.data_ptr(), x.numel(), part.data_ptr(), out.data_ptr(), int(accumulate), _lib.stream())
    return out


def scale_(x: torch.Tensor, scale: float = 1.0, scale_tensor: torch.Tensor | None = None) -> torch.Tensor:
    """x *= scale * (scale_tensor[0] if given); no host sync when the factor lives on the device."""
    if not x.is_cuda:
        x.mul_(scale * (float(scale_tensor[0]) if scale_tensor is not None else 1.0))
        return x
    _lib.call("areno_scale_f32", x.data_ptr(), x.numel(), _lib.ptr(scale_tensor), float(scale), _lib.stream())
    return x
