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


def sample(logits, temperature: float = 1.0, top_k: int = -1, top_p: float = 1.0, *, cls=None, gen_count=None,
           min_new: int = 0, seed: int = 0, row_uid=None, vocab_start: int = 0, out_token=None, out_logprob=None,
           part=None, generator=None):
    """Returns ``(token_ids int64 [B], logprobs fp32 [B])``; with ``part`` (fp32 [B, 6]) writes the
    shard-local candidate record instead (see ``combine_shards``)."""
    if not logits.is_cuda:
        if generator is None and row_uid is not None and temperature > 0.0:
            # counter-based like the kernel: the draw depends only on (seed, row stream, step)
            toks, lps = [], []
            for i in range(logits.shape[0]):
                step = int(gen_count[i]) if gen_count is not None else 0
                g = torch.Generator().manual_seed((int(seed) * 0x9E3779B1 + int(row_uid[i]) * 0x85EBCA77 + step) % (1 << 63))
                t, l = sample_reference(logits[i:i + 1], temperature, top_k, top_p, cls,
                                        None if gen_count is None else gen_count[i:i + 1], min_new, g)
                toks.append(t)
                lps.append(l)
            tok, lp = torch.cat(toks), torch.cat(lps)
        else:
            tok, lp = sample_reference(logits, temperature, top_k, top_p, cls, gen_count, min_new, generator)
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
    _lib.call(
        "areno_sample", logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0), b, v, vocab_start,
        _lib.ptr(cls), _lib.ptr(gen_count), int(min_new), float(temperature), int(top_k if top_k else -1),
        float(top_p), int(seed), _lib.ptr(row_uid), _lib.ptr(out_token), _lib.ptr(out_logprob), _lib.ptr(part),
        _lib.stream(),
    )
    return out_token, out_logprob


def combine_shards(parts: torch.Tensor):
    """parts: fp32 ``[tp, B, 6]`` gathered candidate records -> (tokens int64 [B], logprobs fp32 [B])."""
    best = parts[:, :, 0].argmax(0)
    idx = best[None, :, None].expand(1, -1, 6)
    win = parts.gather(0, idx).squeeze(0)
    tokens = win[:, 1].contiguous().view(torch.int32).to(torch.int64)
    gmax = parts[:, :, 3].max(0).values
    total = (parts[:, :, 4] * torch.exp(parts[:, :, 3] - gmax[None, :])).sum(0)
    return tokens, win[:, 2] - (gmax + torch.log(total))
