"""Decode-time sampler: greedy / temperature / top-k / top-p with suppression and min-new-tokens.

The CUDA path is a single kernel per step that also returns the raw-logit log-probability of
the chosen token (temperature 1, no truncation), so rollout log-probs cost no extra pass.
Noise is counter-based (Philox keyed on seed, row uid, step and global token id): the same call
on vocabulary shards held by different TP ranks draws consistent noise, and ``combine_shards``
merges their candidates.

Counterpart of ``areno/engine/data/sampling.py:26-196`` in the reference.
"""

from __future__ import annotations

import torch

from . import _lib

CLS_NORMAL, CLS_SUPPRESS, CLS_EOS = 0, 1, 2


def build_token_classes(vocab_size: int, suppress_ids=(), eos_ids=(), device="cpu") -> torch.Tensor:
    """int8 ``[vocab]`` table: 1 = never sampled, 2 = EOS-like (masked while step < min_new_tokens)."""
    cls = torch.zeros(vocab_size, dtype=torch.int8)
    for t in eos_ids:
        if 0 <= int(t) < vocab_size:
            cls[int(t)] = CLS_EOS
    for t in suppress_ids:
        if 0 <= int(t) < vocab_size:
            cls[int(t)] = CLS_SUPPRESS
    return cls.to(device)


def sample_reference(logits, temperature, top_k, top_p, cls=None, gen_count=None, min_new=0, generator=None):
    """PyTorch restatement (sort-based) used on CPU and as a distribution oracle."""
    raw = logits.float()
    scores = torch.nan_to_num(raw, nan=float("-inf"), posinf=torch.finfo(torch.float32).max, neginf=float("-inf"))
    if cls is not None:
        c = cls.to(scores.device)
        scores = scores.masked_fill((c == CLS_SUPPRESS)[None, :], float("-inf"))
        if gen_count is not None and min_new > 0:
            early = (gen_count.to(scores.device) < min_new)[:, None] & (c == CLS_EOS)[None, :]
            scores = scores.masked_fill(early, float("-inf"))
    if temperature <= 0.0:
        tok = scores.argmax(-1)
    else:
        probs = torch.softmax(scores / temperature, -1)
        if top_k > 0 or top_p < 1.0:
            ps, pi = probs.sort(-1, descending=True)
            if top_k > 0:
                ps[:, min(top_k, ps.shape[-1]):] = 0.0
            if top_p < 1.0:
                cs = ps.cumsum(-1)
                ps[(cs - ps) > top_p] = 0.0
            ps = ps / ps.sum(-1, keepdim=True).clamp_min(1e-30)
            tok = pi.gather(-1, torch.multinomial(ps, 1, generator=generator)).squeeze(-1)
        else:
            tok = torch.multinomial(probs, 1, generator=generator).squeeze(-1)
    lp = torch.log_softmax(torch.nan_to_num(raw, nan=float("-inf")), -1).gather(-1, tok[:, None]).squeeze(-1)
    return tok, lp


def _s64(x: int) -> int:
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


def _lsr(x: torch.Tensor, n: int) -> torch.Tensor:
    return (x >> n) & ((1 << (64 - n)) - 1)


def _keyed_uniform(seed: int, uid: torch.Tensor, step: torch.Tensor, gidx: torch.Tensor) -> torch.Tensor:
    """Counter-based uniforms in (0, 1): a pure function of (seed, row stream, step, global token id),
    so vocabulary shards on different ranks draw consistent noise (splitmix64 finaliser)."""
    x = (uid.to(torch.int64)[:, None] * _s64(0x9E3779B97F4A7C15) + step.to(torch.int64)[:, None] * _s64(0xD1B54A32D192ED03)
         + gidx.to(torch.int64)[None, :] * _s64(0x8CB92BA72F3D8DD7) + _s64(int(seed) * 0xA0761D6478BD642F))
    x = (x ^ _lsr(x, 30)) * _s64(0xBF58476D1CE4E5B9)
    x = (x ^ _lsr(x, 27)) * _s64(0x94D049BB133111EB)
    x = x ^ _lsr(x, 31)
    u = (_lsr(x, 11).to(torch.float64) + 0.5) / float(1 << 53)
    return u


def sample_keyed_reference(logits, temperature, top_k, top_p, cls=None, gen_count=None, min_new=0, seed=0,
                           row_uid=None, vocab_start=0):
    """CPU counterpart of the sampling kernel: Gumbel-max with counter-based noise.  Returns the
    candidate record ``[B, 6]`` = (best perturbed score, global token id bits, raw logit of the
    winner, raw max, raw sum-exp relative to the max, 0); ``combine_shards`` finishes it."""
    raw = logits.float()
    b, v = raw.shape
    scores = torch.where(torch.isnan(raw), torch.full_like(raw, float("-inf")), raw)
    if cls is not None:
        c = cls.to(raw.device)[vocab_start:vocab_start + v]
        scores = scores.masked_fill((c == CLS_SUPPRESS)[None, :], float("-inf"))
        if gen_count is not None and min_new > 0:
            early = (gen_count.to(raw.device) < min_new)[:, None] & (c == CLS_EOS)[None, :]
            scores = scores.masked_fill(early, float("-inf"))
    greedy = temperature <= 0.0
    if not greedy and (top_k > 0 or top_p < 1.0):
        probs = torch.softmax(scores / temperature, -1)
        ps, pi = probs.sort(-1, descending=True)
        keep_sorted = torch.ones_like(ps, dtype=torch.bool)
        if top_k > 0:
            keep_sorted[:, min(top_k, v):] = False
        if top_p < 1.0:
            keep_sorted &= (ps.cumsum(-1) - ps) <= top_p
        keep = torch.zeros_like(keep_sorted).scatter(1, pi, keep_sorted)
        scores = scores.masked_fill(~keep, float("-inf"))
    if greedy:
        pert = scores
    else:
        uid = row_uid if row_uid is not None else torch.arange(b)
        step = gen_count if gen_count is not None else torch.zeros(b, dtype=torch.int64)
        u = _keyed_uniform(seed, uid.cpu(), step.cpu(), vocab_start + torch.arange(v))
        pert = scores / temperature + (-torch.log(-torch.log(u))).to(torch.float32)
    bv, bi = pert.max(-1)
    finite = torch.where(torch.isnan(raw), torch.full_like(raw, float("-inf")), raw).clamp(max=3.0e38)
    m = finite.max(-1).values
    ssum = torch.exp(finite - m[:, None]).sum(-1)
    rec = torch.zeros((b, 6), dtype=torch.float32)
    rec[:, 0] = bv
    rec[:, 1] = (vocab_start + bi).to(torch.int32).view(torch.float32)
    rec[:, 2] = raw.gather(-1, bi[:, None]).squeeze(-1)
    rec[:, 3] = m
    rec[:, 4] = ssum
    return rec



def sample(logits, temperature: float = 1.0, top_k: int = -1, top_p: float = 1.0, *, cls=None, gen_count=None,
           min_new: int = 0, seed: int = 0, row_uid=None, vocab_start: int = 0, out_token=None, out_logprob=None,
           part=None, generator=None):
    """Returns ``(token_ids int64 [B], logprobs fp32 [B])``; with ``part`` (fp32 [B, 6]) writes the
    shard-local candidate record instead (see ``combine_shards``)."""
    if not logits.is_cuda:
        if generator is not None:
            tok, lp = sample_reference(logits, temperature, top_k, top_p, cls, gen_count, min_new, generator)
        else:
            rec = sample_keyed_reference(logits, temperature, top_k, top_p, cls, gen_count, min_new, seed, row_uid,
                                         vocab_start)
            if part is not None:
                part.copy_(rec)
                return None, None
            tok, lp = combine_shards(rec[None])
        if out_token is not None:
            out_token.copy_(tok)
            tok = out_token
        if out_logprob is not None:
            out_logprob.copy_(lp)
            lp = out_logprob
        return tok, lp
    b, v = logits.shape
    assert logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    if out_token is None and part is None:
        out_token = torch.empty(b, dtype=torch.int64, device=logits.device)
    if out_logprob is None and part is None:
        out_logprob = torch.empty(b, dtype=torch.float32, device=logits.device)
    # few rows, long vocabulary: several blocks per row (vocabulary slices), winner picked by a second kernel
    slices = 0 if b * 2 > 148 else min(16, max(1, 296 // max(b, 1)))
    scratch = _slice_scratch(logits.device, slices * b * 6) if slices > 1 else None
    _lib.call(
        "areno_sample", logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0), b, v, vocab_start,
        _lib.ptr(cls), _lib.ptr(gen_count), int(min_new), float(temperature), int(top_k if top_k else -1),
        float(top_p), int(seed), _lib.ptr(row_uid), _lib.ptr(out_token), _lib.ptr(out_logprob), _lib.ptr(part),
        _lib.ptr(scratch), int(slices), _lib.stream(),
    )
    return out_token, out_logprob


_SLICE_SCRATCH: dict = {}
_RETIRED: list = []


def _slice_scratch(device, elems: int) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _SLICE_SCRATCH.get(key)
    if buf is None or buf.numel() < elems:
        if buf is not None:
            _RETIRED.append(buf)      # captured decode graphs may still point at the outgrown buffer
        buf = torch.empty(max(elems, 16 * 148 * 6), dtype=torch.float32, device=device)
        _SLICE_SCRATCH[key] = buf
    return buf


def combine_shards(parts: torch.Tensor):
    """parts: fp32 ``[tp, B, 6]`` gathered candidate records -> (tokens int64 [B], logprobs fp32 [B])."""
    best = parts[:, :, 0].argmax(0)
    idx = best[None, :, None].expand(1, -1, 6)
    win = parts.gather(0, idx).squeeze(0)
    tokens = win[:, 1].contiguous().view(torch.int32).to(torch.int64)
    gmax = parts[:, :, 3].max(0).values
    total = (parts[:, :, 4] * torch.exp(parts[:, :, 3] - gmax[None, :])).sum(0)
    return tokens, win[:, 2] - (gmax + torch.log(total))
