"""Ops of the hybrid (linear-attention) layers: causal depthwise conv1d + SiLU, the gated delta rule,
RMSNorm with a SiLU gate, decayed linear ("lightning") attention with forward and backward kernels, and
group RMSNorm with a sigmoid gate.

Inference (prefill and decode) runs the CUDA kernels of ``csrc/linear_attn.cu`` with per-slot conv
and recurrent-state caches.  Training uses the CUDA conv / gated-norm kernels (forward and backward);
the gated delta rule itself is differentiated through a chunk-parallel PyTorch formulation
(``gated_delta_rule_chunked``): its backward has no hand-written kernel yet.  The recurrent PyTorch
version (``gated_delta_rule_reference``) is the oracle for both.

Reference roles: ``areno/accel/csrc/conv.cu``, ``normalization.cu:84-178`` and the FLA kernels wrapped
in ``areno/models/_shared/dynamo_wrappers.py:16-104``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib

_lib.register_signature("areno_conv1d_silu_fwd", "plppppliiplp")
_lib.register_signature("areno_conv1d_silu_bwd_blocks", "l")
_lib.register_signature("areno_conv1d_silu_bwd", "plpppplliiplpp")
_lib.register_signature("areno_conv1d_update_hist", "plpppiiipp")
_lib.register_signature("areno_conv1d_silu_decode", "plppiiipplp")
_lib.register_signature("areno_gdn_recurrent", "pplplpppppppiiiiifplp")
_lib.register_signature("areno_lightning_recurrent", "ppplppppppiiifplp")
_lib.register_signature("areno_lightning_bwd", "ppplplppiiifppplp")
_lib.register_signature("areno_group_rmsnorm_gate_fwd", "pplpliifppp")
_lib.register_signature("areno_group_rmsnorm_gate_dw_blocks", "l")
_lib.register_signature("areno_group_rmsnorm_gate_bwd", "ppplppliipppp")
_lib.register_signature("areno_rmsnorm_silu_gate_fwd", "ppliplifppp")
_lib.register_signature("areno_rmsnorm_silu_gate_bwd_blocks", "l")
_lib.register_signature("areno_rmsnorm_silu_gate_bwd", "ppplipplipplpp")


# ------------------------------------------------------------------------------ helpers
def seq_index_tensors(lens: list[int], device):
    """``(seq_start, seq_end, seq_id, cu)`` int32 tensors for packed rows of the given lengths."""
    starts, ends, ids, cu, off = [], [], [], [0], 0
    for i, n in enumerate(lens):
        starts += [off] * n
        ends += [off + n] * n
        ids += [i] * n
        off += n
        cu.append(off)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return mk(starts), mk(ends), mk(ids), mk(cu)


# --------------------------------------------------------------------------------- conv
def conv1d_silu_reference(x, w, lens, hist=None):
    """x: [T, C]; w: [C, K] fp32; hist: optional [num_seqs, C, K-1] inputs preceding each sequence."""
    k = w.shape[1]
    outs, off = [], 0
    for i, n in enumerate(lens):
        seg = x[off:off + n].float()
        pad = hist[i].t().float() if hist is not None else torch.zeros(k - 1, x.shape[1], dtype=torch.float32, device=x.device)
        full = torch.cat([pad, seg], 0)                      # [K-1+n, C]
        win = full.unfold(0, k, 1)                           # [n, C, K]
        outs.append(F.silu((win * w.float()[None]).sum(-1)))
        off += n
    return torch.cat(outs, 0).to(x.dtype) if outs else x.new_zeros(x.shape)


class _ConvSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, idx, hist):
        seq_start, seq_end, seq_id, _cu = idx
        t, c = x.shape
        k = w.shape[1]
        y = torch.empty((t, c), dtype=x.dtype, device=x.device)
        _lib.call("areno_conv1d_silu_fwd", x.data_ptr(), x.stride(0), w.data_ptr(), seq_start.data_ptr(),
                  seq_id.data_ptr(), _lib.ptr(hist), t, c, k, y.data_ptr(), y.stride(0), _lib.stream())
        ctx.save_for_backward(x, w)
        ctx.idx = idx
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        seq_start, seq_end, _sid, _cu = ctx.idx
        t, c = x.shape
        k = w.shape[1]
        if dy.stride(1) != 1:
            dy = dy.contiguous()
        dx = torch.empty((t, c), dtype=x.dtype, device=x.device)
        nblk = _lib.fn("areno_conv1d_silu_bwd_blocks")(t)
        part = torch.empty((nblk, c, k), dtype=torch.float32, device=x.device)
        _lib.call("areno_conv1d_silu_bwd", x.data_ptr(), x.stride(0), w.data_ptr(), seq_start.data_ptr(),
                  seq_end.data_ptr(), dy.data_ptr(), dy.stride(0), t, c, k, dx.data_ptr(), dx.stride(0), part.data_ptr(),
                  _lib.stream())
        return dx, part.sum(0), None, None


def conv1d_silu(x, w, lens, idx=None, hist=None):
    """Depthwise causal conv + SiLU over packed rows ``x [T, C]`` (column stride 1, any row stride)."""
    if not x.is_cuda:
        return conv1d_silu_reference(x, w, lens, hist)
    if idx is None:
        idx = seq_index_tensors(lens, x.device)
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.dtype == torch.float32 and w.is_contiguous()
    return _ConvSilu.apply(x, w, idx, hist)


def conv1d_update_hist(x, cu, slots, fresh, hist_cache, k: int):
    """Store the last ``K-1`` inputs of every sequence of a prefill chunk into ``hist_cache[slot]``."""
    n = slots.numel()
    if not x.is_cuda:
        cu_l = cu.tolist()
        for i in range(n):
            seg = x[cu_l[i]:cu_l[i + 1]].float()
            old = torch.zeros_like(hist_cache[0]) if bool(fresh[i]) else hist_cache[int(slots[i])].clone()
            full = torch.cat([old.t(), seg], 0)
            hist_cache[int(slots[i])] = full[-(k - 1):].t()
        return
    _lib.call("areno_conv1d_update_hist", x.data_ptr(), x.stride(0), cu.data_ptr(), slots.data_ptr(), _lib.ptr(fresh), n,
              x.shape[1], k, hist_cache.data_ptr(), _lib.stream())


def conv1d_silu_decode(x, w, hist_cache, active=None):
    """One new row per slot (row i <-> slot i); updates ``hist_cache`` in place for active rows."""
    rows, c = x.shape
    k = w.shape[1]
    if not x.is_cuda:
        win = torch.cat([hist_cache[:rows].float(), x.float()[:, :, None]], -1)          # [rows, C, K]
        y = F.silu((win * w.float()[None]).sum(-1)).to(x.dtype)
        keep = torch.ones(rows, dtype=torch.bool) if active is None else active[:rows] > 0
        hist_cache[:rows][keep] = win[keep][:, :, 1:]
        return y
    y = torch.empty((rows, c), dtype=x.dtype, device=x.device)
    _lib.call("areno_conv1d_silu_decode", x.data_ptr(), x.stride(0), w.data_ptr(), _lib.ptr(active), rows, c, k,
              hist_cache.data_ptr(), y.data_ptr(), y.stride(0), _lib.stream())
    return y


# ---------------------------------------------------------------------- gated delta rule
def gated_delta_rule_reference(q, k, v, g, beta, lens, scale, state=None):
    """Token-by-token recurrence in fp32.  q, k: [T, Hk, DK] (already l2-normalised); v: [T, Hv, DV];
    g, beta: [T, Hv].  ``state``: optional list of per-sequence initial states [Hv, DK, DV]; returns
    ``(out [T, Hv, DV], final_states)``."""
    t, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    rep = hv // hk
    qf = q.float().repeat_interleave(rep, 1)
    kf = k.float().repeat_interleave(rep, 1)
    vf, gf, bf = v.float(), g.float(), beta.float()
    out = torch.zeros((t, hv, dv), dtype=torch.float32, device=q.device)
    finals, off = [], 0
    for i, n in enumerate(lens):
        s = state[i].float().clone() if state is not None else torch.zeros((hv, dk, dv), dtype=torch.float32, device=q.device)
        for r in range(off, off + n):
            s = s * torch.exp(gf[r])[:, None, None]
            u = torch.einsum("hk,hkv->hv", kf[r], s)
            d = bf[r][:, None] * (vf[r] - u)
            s = s + kf[r][:, :, None] * d[:, None, :]
            out[r] = torch.einsum("hk,hkv->hv", qf[r], s) * scale
        finals.append(s)
        off += n
    return out.to(v.dtype), finals


def gated_delta_rule_chunked(q, k, v, g, beta, lens, scale, chunk: int = 64):
    """Chunk-parallel formulation (WY representation) in PyTorch, differentiable by autograd; used for
    training.  Same inputs as the reference; returns ``out [T, Hv, DV]``."""
    t, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    rep = hv // hk
    outs, off = [], 0
    for n in lens:
        sl = slice(off, off + n)
        qs = q[sl].float().repeat_interleave(rep, 1).transpose(0, 1) * scale      # [H, n, dk]
        ks = k[sl].float().repeat_interleave(rep, 1).transpose(0, 1)
        vs = v[sl].float().transpose(0, 1)                                          # [H, n, dv]
        gs = g[sl].float().transpose(0, 1)                                          # [H, n]
        bs = beta[sl].float().transpose(0, 1)
        pad = (-n) % chunk
        if pad:
            qs, ks, vs = (F.pad(x, (0, 0, 0, pad)) for x in (qs, ks, vs))
            gs, bs = F.pad(gs, (0, pad)), F.pad(bs, (0, pad))
        L = n + pad
        nc = L // chunk
        qs, ks, vs = (x.reshape(hv, nc, chunk, -1) for x in (qs, ks, vs))
        gs, bs = gs.reshape(hv, nc, chunk), bs.reshape(hv, nc, chunk)
        gc = gs.cumsum(-1)                                                          # within-chunk log decay
        kb, vb = ks * bs[..., None], vs * bs[..., None]
        decay = torch.exp((gc[..., :, None] - gc[..., None, :]).tril())
        strict = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), -1)
        incl = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), 0)
        a = -(kb @ ks.transpose(-1, -2) * decay).masked_fill(~strict, 0)
        # (I - A)^-1 by forward substitution over rows
        rows = [a[..., 0, :]]
        for i in range(1, chunk):
            row = a[..., i, :] + (a[..., i, :i, None] * torch.stack(rows, -2)[..., :i, :]).sum(-2)
            rows.append(row)
        tmat = torch.stack(rows, -2) + torch.eye(chunk, device=q.device)
        w_ = tmat @ (kb * torch.exp(gc)[..., None])
        u_ = tmat @ vb
        s = torch.zeros((hv, dk, dv), dtype=torch.float32, device=q.device)
        o_chunks = []
        for c in range(nc):
            qc, kc, gcc = qs[:, c], ks[:, c], gc[:, c]
            attn = (qc @ kc.transpose(-1, -2) * decay[:, c]).masked_fill(~incl, 0)
            v_new = u_[:, c] - w_[:, c] @ s
            o_chunks.append((qc * torch.exp(gcc)[..., None]) @ s + attn @ v_new)
            last = gcc[:, -1]
            s = s * torch.exp(last)[:, None, None] + (kc * torch.exp(last[:, None] - gcc)[..., None]).transpose(-1, -2) @ v_new
        o = torch.stack(o_chunks, 1).reshape(hv, L, dv)[:, :n]
        outs.append(o.transpose(0, 1))
        off += n
    return torch.cat(outs, 0).to(v.dtype)


def gated_delta_rule_recurrent(q, k, v, g, beta, cu, scale, *, state_cache=None, slots=None, fresh=None, active=None):
    """CUDA recurrence for inference.  ``q`` / ``k``: [T, Hk, DK] views with unit stride on DK and head
    stride DK (row stride free, shared by q and k); ``v``: [T, Hv, DV].  ``state_cache`` fp32
    [slots, Hv, DK, DV] is read (unless ``fresh[seq]``) and written in place."""
    t, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    num_seqs = cu.numel() - 1
    assert q.stride(0) == k.stride(0) and q.stride(2) == 1 and q.stride(1) == dk and v.stride(2) == 1 and v.stride(1) == dv
    out = torch.empty((t, hv, dv), dtype=v.dtype, device=v.device)
    _lib.call("areno_gdn_recurrent", q.data_ptr(), k.data_ptr(), q.stride(0), v.data_ptr(), v.stride(0),
              g.contiguous().data_ptr(), beta.contiguous().data_ptr(), cu.data_ptr(), _lib.ptr(slots), _lib.ptr(fresh),
              _lib.ptr(active), _lib.ptr(state_cache), num_seqs, hk, hv, dk, dv, float(scale), out.data_ptr(),
              out.stride(0), _lib.stream())
    return out


# ------------------------------------------------------------------- rmsnorm * silu(gate)
def rmsnorm_silu_gate_reference(x, gate, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return (y * F.silu(gate.float())).to(x.dtype)


class _RmsnormSiluGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, w, eps):
        # x: [T, H, D] contiguous; gate: [T, H, D] view (unit stride on D, head stride D, any token stride)
        t, h, d = x.shape
        rows = t * h
        y = torch.empty_like(x)
        inv = torch.empty(rows, dtype=torch.float32, device=x.device)
        _lib.call("areno_rmsnorm_silu_gate_fwd", x.data_ptr(), gate.data_ptr(), gate.stride(0), h, w.data_ptr(), rows, d,
                  float(eps), y.data_ptr(), inv.data_ptr(), _lib.stream())
        ctx.save_for_backward(x, gate, w, inv)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gate, w, inv = ctx.saved_tensors
        t, h, d = x.shape
        rows = t * h
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dgate = torch.empty((t, h, d), dtype=x.dtype, device=x.device)
        nblk = _lib.fn("areno_rmsnorm_silu_gate_bwd_blocks")(rows)
        part = torch.empty((nblk, d), dtype=torch.float32, device=x.device)
        _lib.call("areno_rmsnorm_silu_gate_bwd", dy.data_ptr(), x.data_ptr(), gate.data_ptr(), gate.stride(0), h,
                  w.data_ptr(), inv.data_ptr(), rows, d, dx.data_ptr(), dgate.data_ptr(), dgate.stride(0), part.data_ptr(),
                  _lib.stream())
        return dx, dgate, part.sum(0).to(w.dtype), None


def rmsnorm_silu_gate(x, gate, w, eps: float):
    """``rmsnorm(x) * w * silu(gate)`` over the last dim of ``x [T, H, D]`` (``w`` fp32 [D])."""
    if not x.is_cuda:
        return rmsnorm_silu_gate_reference(x, gate, w, eps)
    assert x.is_contiguous() and gate.stride(2) == 1 and gate.stride(1) == x.shape[2] and w.dtype == torch.float32
    return _RmsnormSiluGate.apply(x, gate, w, float(eps))


# ---------------------------------------------------------------- decayed linear attention
def lightning_attention_reference(q, k, v, slope, lens, scale, state=None):
    """``S_t = exp(-slope_h) S_{t-1} + k_t v_t^T``, ``o_t = scale q_t^T S_t`` per sequence, in fp32 PyTorch
    (differentiable).  ``q, k, v``: [T, H, D]; ``slope``: [H]; ``state``: optional list of [H, D, D] start
    states.  Returns ``(out [T, H, D], final states)``.  Semantics of the reference's
    ``chunk_lightning_attn`` / ``seg_la_fwd`` calls (``areno/models/bailing/model.py:904-1003``)."""
    decay = torch.exp(-slope.float())[:, None, None]
    outs, finals, off = [], [], 0
    for i, n in enumerate(lens):
        s = torch.zeros((q.shape[1], q.shape[2], v.shape[2]), dtype=torch.float32, device=q.device) \
            if state is None or state[i] is None else state[i].float()
        for t in range(off, off + n):
            s = decay * s + k[t].float()[:, :, None] * v[t].float()[:, None, :]
            outs.append(torch.einsum("hd,hde->he", q[t].float(), s) * scale)
        finals.append(s)
        off += n
    out = torch.stack(outs, 0) if outs else torch.zeros_like(v, dtype=torch.float32)
    return out.to(v.dtype), finals


def _same_layout(q, k, v):
    d = q.shape[2]
    return all(x.stride(2) == 1 and x.stride(1) == d and x.stride(0) == q.stride(0) and x.shape == q.shape for x in (q, k, v))


def lightning_recurrent(q, k, v, slope, cu, scale, *, state_cache=None, slots=None, fresh=None, active=None):
    """CUDA scan (inference prefill chunks, decode rows, training forward).  ``q, k, v``: [T, H, D] views
    with one shared row stride; ``state_cache`` fp32 [slots, H, D, D] is read unless ``fresh[seq]`` and
    written in place."""
    assert _same_layout(q, k, v) and q.dtype == torch.bfloat16
    t, h, d = q.shape
    out = torch.empty((t, h, d), dtype=q.dtype, device=q.device)
    log_decay = (-slope.float()).contiguous()
    _lib.call("areno_lightning_recurrent", q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), log_decay.data_ptr(),
              cu.data_ptr(), _lib.ptr(slots), _lib.ptr(fresh), _lib.ptr(active), _lib.ptr(state_cache), cu.numel() - 1,
              h, d, float(scale), out.data_ptr(), out.stride(0), _lib.stream())
    return out


class _Lightning(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, slope, cu, scale):
        out = lightning_recurrent(q, k, v, slope, cu, scale)
        ctx.save_for_backward(q, k, v, slope, cu)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, slope, cu = ctx.saved_tensors
        t, h, d = q.shape
        d_o = d_o.contiguous()
        grads = torch.empty((3, t, h, d), dtype=q.dtype, device=q.device)
        _lib.call("areno_lightning_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), d_o.data_ptr(),
                  d_o.stride(0), slope.data_ptr(), cu.data_ptr(), cu.numel() - 1, h, d, float(ctx.scale),
                  grads[0].data_ptr(), grads[1].data_ptr(), grads[2].data_ptr(), grads.stride(1), _lib.stream())
        return grads[0], grads[1], grads[2], None, None, None


def lightning_attention(q, k, v, slope, lens, scale, cu=None):
    """Differentiable decayed linear attention over packed sequences (training).  ``slope`` fp32 [H]."""
    if not q.is_cuda:
        return lightning_attention_reference(q, k, v, slope, lens, scale)[0]
    if cu is None:
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32, device=q.device)
    if not _same_layout(q, k, v):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    return _Lightning.apply(q, k, v, slope.float().contiguous(), cu, float(scale))


# -------------------------------------------------------------- group rmsnorm * sigmoid(gate)
def group_rmsnorm_sigmoid_gate_reference(x, gate, w, eps):
    g, width = w.shape
    xf = x.float().unflatten(-1, (g, width))
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return (y.flatten(-2) * torch.sigmoid(gate.float())).to(x.dtype)


class _GroupNormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, w, eps):
        rows = x.shape[0]
        g, width = w.shape
        y = torch.empty_like(x)
        inv = torch.empty(rows * g, dtype=torch.float32, device=x.device)
        _lib.call("areno_group_rmsnorm_gate_fwd", x.data_ptr(), gate.data_ptr(), gate.stride(0), w.data_ptr(), rows, g,
                  width, float(eps), y.data_ptr(), inv.data_ptr(), _lib.stream())
        ctx.save_for_backward(x, gate, w, inv)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gate, w, inv = ctx.saved_tensors
        rows = x.shape[0]
        g, width = w.shape
        dy = dy.contiguous()
        dx, dgate = torch.empty_like(x), torch.empty_like(x)
        nblk = _lib.fn("areno_group_rmsnorm_gate_dw_blocks")(rows)
        part = torch.empty((nblk, g * width), dtype=torch.float32, device=x.device)
        _lib.call("areno_group_rmsnorm_gate_bwd", dy.data_ptr(), x.data_ptr(), gate.data_ptr(), gate.stride(0),
                  w.data_ptr(), inv.data_ptr(), rows, g, width, dx.data_ptr(), dgate.data_ptr(), part.data_ptr(),
                  _lib.stream())
        return dx, dgate, part.sum(0).view(g, width).to(w.dtype), None


def group_rmsnorm_sigmoid_gate(x, gate, w, eps: float):
    """``x [T, G*W]`` (contiguous) normalised per group of ``W`` channels, scaled by ``w`` (fp32 [G, W]) and
    multiplied by ``sigmoid(gate)``; ``gate [T, G*W]`` may have any row stride.  Role of
    ``GroupRMSNormSigmoidGate`` (``areno/engine/layers/norm.py:60-105``)."""
    if not x.is_cuda:
        return group_rmsnorm_sigmoid_gate_reference(x, gate, w, eps)
    assert x.is_contiguous() and gate.stride(1) == 1 and w.dtype == torch.float32 and w.is_contiguous()
    return _GroupNormGate.apply(x, gate, w, float(eps))
