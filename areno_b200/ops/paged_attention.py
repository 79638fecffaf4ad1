"""Paged KV cache ops: RoPE + append, and decode attention over bf16 or fp8-e4m3 pages.

Cache layout per layer: ``k_cache``/``v_cache`` of shape ``[num_pages, kv_heads, PAGE, head_dim]``
(bf16, or uint8 holding e4m3 with fp32 ``k_scale``/``v_scale`` of shape ``[num_pages, kv_heads, PAGE]``).
``PAGE`` is fixed by the kernels (64 tokens).  A token's global slot is ``page * PAGE + offset``.

Replaces ``flash_attn_with_kvcache`` and the index_put KV scatter of the reference
(``areno/engine/layers/attention_backend/infer.py:138-178``).
"""

from __future__ import annotations

import os

import torch

from . import _lib
from .rope import rope_reference

PAGE = 64


def alloc_kv_cache(num_pages: int, kv_heads: int, head_dim: int, device, fp8: bool = False):
    """Returns (k_cache, v_cache, k_scale, v_scale); scales are None for bf16 pages."""
    shape = (num_pages, kv_heads, PAGE, head_dim)
    if fp8:
        k = torch.zeros(shape, dtype=torch.uint8, device=device)
        v = torch.zeros(shape, dtype=torch.uint8, device=device)
        ks = torch.ones((num_pages, kv_heads, PAGE), dtype=torch.float32, device=device)
        vs = torch.ones((num_pages, kv_heads, PAGE), dtype=torch.float32, device=device)
        return k, v, ks, vs
    return (torch.zeros(shape, dtype=torch.bfloat16, device=device),
            torch.zeros(shape, dtype=torch.bfloat16, device=device), None, None)


def _quant_e4m3_reference(x):
    amax = x.float().abs().amax(-1, keepdim=True).clamp_min(1e-8)
    scale = amax / 448.0
    q = (x.float() / scale).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), scale.squeeze(-1)


def rope_append_kv(qkv, positions, slot_mapping, k_cache, v_cache, k_scale, v_scale, hq, hkv, d,
                   theta=10000.0, rot_dim=None, inv_freq=None, interleaved=False):
    """In place: rotate the q and k parts of ``qkv`` ([T, (hq+2hkv)*d]) and write k, v into the cache
    at ``slot_mapping`` (int32, negative = skip)."""
    rot = d if rot_dim is None else rot_dim
    fp8 = k_cache.dtype == torch.uint8
    if not qkv.is_cuda:
        t = qkv.shape[0]
        q = qkv[:, : hq * d].view(t, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].view(t, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(t, hkv, d)
        if rot > 0:
            q.copy_(rope_reference(q, positions, theta, rot, inv_freq, interleaved))
            k.copy_(rope_reference(k, positions, theta, rot, inv_freq, interleaved))
        valid = slot_mapping >= 0
        pages = (slot_mapping[valid] // PAGE).long()
        offs = (slot_mapping[valid] % PAGE).long()
        if fp8:
            kq, ks = _quant_e4m3_reference(k[valid])
            vq, vs = _quant_e4m3_reference(v[valid])
            k_cache[pages, :, offs] = kq
            v_cache[pages, :, offs] = vq
            k_scale[pages, :, offs] = ks
            v_scale[pages, :, offs] = vs
        else:
            k_cache[pages, :, offs] = k[valid].to(k_cache.dtype)
            v_cache[pages, :, offs] = v[valid].to(v_cache.dtype)
        return qkv
    assert qkv.is_contiguous() and qkv.dtype == torch.bfloat16
    if positions.dtype != torch.int32:
        positions = positions.to(torch.int32)
    if slot_mapping.dtype != torch.int32:
        slot_mapping = slot_mapping.to(torch.int32)
    _lib.check_index("rope_append_kv slot_mapping", slot_mapping, k_cache.shape[0] * PAGE, low=-1)
    _lib.call(
        "areno_rope_append_kv", qkv.data_ptr(), positions.data_ptr(), slot_mapping.data_ptr(), _lib.ptr(inv_freq),
        k_cache.data_ptr(), v_cache.data_ptr(), _lib.ptr(k_scale), _lib.ptr(v_scale), qkv.shape[0], hq, hkv, d, rot,
        float(theta), int(interleaved), PAGE, int(fp8), _lib.stream(),
    )
    return qkv


def _dequant(cache, scale):
    if cache.dtype != torch.uint8:
        return cache.float()
    return cache.view(torch.float8_e4m3fn).float() * scale.unsqueeze(-1)


def fold_rope_append_kv(part, bias, positions, slot_mapping, k_cache, v_cache, k_scale, v_scale, hq, hkv, d,
                        theta=10000.0, rot_dim=None, inv_freq=None, interleaved=False, q_norm_w=None, k_norm_w=None,
                        norm_eps: float = 1e-6, norm_offset: float = 0.0):
    """Decode-sized q/k/v projection left as split-K partials (``ops.gemm.SplitKPartial``): fold + bias +
    optional per-head q / k RMSNorm + rotary embedding + KV append in one launch.  Returns the bf16
    ``[T, (hq + 2 hkv) d]`` tensor (q rotated, k rotated, v), as ``linear`` + head norms + ``rope_append_kv`` would."""
    rot = d if rot_dim is None else rot_dim
    t, n = part.rows, part.n
    assert n == (hq + 2 * hkv) * d
    qkv = torch.empty((t, n), dtype=torch.bfloat16, device=k_cache.device)
    if positions.dtype != torch.int32:
        positions = positions.to(torch.int32)
    if slot_mapping.dtype != torch.int32:
        slot_mapping = slot_mapping.to(torch.int32)
    wf32 = int(q_norm_w is not None and q_norm_w.dtype == torch.float32)
    _lib.check_index("fold_rope_append_kv slot_mapping", slot_mapping, k_cache.shape[0] * PAGE, low=-1)
    _lib.call("areno_fold_rope_append_kv", part.ws.data_ptr(), part.splits, t * n, _lib.ptr(bias), qkv.data_ptr(),
              positions.data_ptr(), slot_mapping.data_ptr(), _lib.ptr(inv_freq), k_cache.data_ptr(), v_cache.data_ptr(),
              _lib.ptr(k_scale), _lib.ptr(v_scale), t, hq, hkv, d, rot, float(theta), int(interleaved), PAGE,
              int(k_cache.dtype == torch.uint8), _lib.ptr(q_norm_w), _lib.ptr(k_norm_w), wf32, float(norm_offset),
              float(norm_eps), _lib.stream())
    return qkv


def paged_decode_reference(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, scale, window=0):
    """q: [B, hq, d] -> [B, hq, d] (fp32 math)."""
    b, hq, d = q.shape
    hkv = k_cache.shape[1]
    group = hq // hkv
    out = torch.zeros((b, hq, d), dtype=torch.float32, device=q.device)
    kc, vc = _dequant(k_cache, k_scale), _dequant(v_cache, v_scale)
    for i in range(b):
        n = int(seq_lens[i])
        if n == 0:
            continue
        npages = (n + PAGE - 1) // PAGE
        pages = block_table[i, :npages].long()
        k = kc[pages].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :n]
        v = vc[pages].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :n]
        k = k.repeat_interleave(group, 0)
        v = v.repeat_interleave(group, 0)
        s = torch.einsum("hd,hnd->hn", q[i].float(), k) * scale
        if window and window > 0:
            idx = torch.arange(n, device=q.device)
            s = s.masked_fill(idx[None, :] < n - window, float("-inf"))
        out[i] = torch.einsum("hn,hnd->hd", torch.softmax(s, -1), v)
    return out.to(q.dtype)


_SCRATCH: dict = {}


# ARENO_DECODE_SPLITS=n forces the number of KV splits of the decode kernel (tuning aid; 0 = heuristic)
_FORCED_SPLITS = int(os.environ.get("ARENO_DECODE_SPLITS", "0") or 0)


def paged_decode(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, scale, max_context: int | None = None,
                 window: int = 0, out=None, scratch=None):
    """Decode attention for one new token per sequence.

    q: ``[B, hq, d]`` (token stride arbitrary); block_table: int32 ``[B, max_pages]``; seq_lens: int32 ``[B]``
    (context length including the token just appended).  ``max_context`` bounds the number of KV
    splits launched (defaults to the block-table capacity); sequences shorter than that simply
    leave the extra CTAs idle, so the launch shape does not depend on device data.
    """
    if not q.is_cuda:
        return paged_decode_reference(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, scale, window)
    b, hq, d = q.shape
    hkv = k_cache.shape[1]
    fp8 = k_cache.dtype == torch.uint8
    max_pages = block_table.shape[1]
    cap_pages = max_pages if max_context is None else min(max_pages, (max_context + PAGE - 1) // PAGE)
    # Split the KV range only as far as it takes to fill the machine (two resident CTAs per SM): with enough
    # (sequence, kv head) pairs every CTA streams its whole context and writes the output itself, and
    # neither partials nor the merge kernel exist.  A split is never shorter than two pages.
    base = b * hkv * ((hq // hkv + 15) // 16)
    want = max(1, min((2 * 148 + base // 2) // base, cap_pages // 2, 32))
    if _FORCED_SPLITS > 0:
        want = max(1, min(_FORCED_SPLITS, cap_pages))
    pages_per_split = (cap_pages + want - 1) // want
    nsplit = (cap_pages + pages_per_split - 1) // pages_per_split
    if out is None:
        out = torch.empty((b, hq, d), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if nsplit > 1:
        if scratch is not None:
            part_o, part_ml = scratch
        else:
            key = (q.device.index, b, hq, nsplit, d)
            sc = _SCRATCH.get(key)
            if sc is None:
                sc = (torch.empty((b, hq, nsplit, d), dtype=torch.float32, device=q.device),
                      torch.empty((b, hq, nsplit, 2), dtype=torch.float32, device=q.device))
                _SCRATCH[key] = sc
            part_o, part_ml = sc
    if _lib.BOUNDS_CHECK:
        _lib.check_index("paged_decode seq_lens", seq_lens, max_pages * PAGE + 1)
        # only the pages below each sequence's length are read: check exactly those entries of the table
        used = (torch.arange(max_pages, device=q.device)[None, :] * PAGE) < seq_lens[:, None]
        _lib.check_index("paged_decode block_table", block_table[used], k_cache.shape[0])
    _lib.call(
        "areno_paged_decode", q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _lib.ptr(k_scale),
        _lib.ptr(v_scale), block_table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), _lib.ptr(part_o),
        _lib.ptr(part_ml), b, hq, hkv, d, max_pages, q.stride(0), out.stride(0), float(scale), pages_per_split, nsplit,
        int(window or 0), int(fp8), _lib.stream(),
    )
    return out
