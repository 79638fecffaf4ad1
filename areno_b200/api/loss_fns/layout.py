"""Uniform view of the response tokens of a training batch, packed or padded.

A loss function receives ``(data_pack, logprobs)``; ``response_layout`` extracts the per-token
signals it needs aligned with ``logprobs`` - flat ``[num_actions]`` vectors for the packed batches
produced by this package's trainer, ``[B, T-1]`` matrices for padded batches from other backends.
Field names and reductions match ``areno/api/loss_fns/layout.py:16-163`` of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class ResponseLayout:
    packed: bool
    response_mask: torch.Tensor      # float {0,1}, same shape as logprobs
    valid_count: torch.Tensor        # scalar, >= 1
    response_len: torch.Tensor       # per-sequence response length (>= 1) or valid_count
    old_logprobs: torch.Tensor | None = None
    advantages: torch.Tensor | None = None
    ref_logprobs: torch.Tensor | None = None
    seq_ids: torch.Tensor | None = None
    num_sequences: int | None = None


def _f32(t: torch.Tensor, device) -> torch.Tensor:
    return t.to(device=device, dtype=torch.float32)


def response_layout(data_pack: dict, logprobs: torch.Tensor, *, need_old_logprobs: bool = False,
                    need_advantages: bool = False, need_ref_logprobs: bool = False,
                    need_sequences: bool = False) -> ResponseLayout:
    dev = logprobs.device
    if "packed_response_mask" in data_pack:
        mask = _f32(data_pack["packed_response_mask"], dev)
        count = mask.sum().clamp(min=1)
        lay = ResponseLayout(packed=True, response_mask=mask, valid_count=count, response_len=count)
        if need_sequences:
            lay.seq_ids = data_pack["packed_seq_ids"].to(device=dev, dtype=torch.long)
            lay.num_sequences = int(data_pack["packed_num_sequences"])
            lens = torch.zeros(lay.num_sequences, device=dev, dtype=torch.float32)
            lens.scatter_add_(0, lay.seq_ids, mask)
            lay.response_len = lens.clamp(min=1)
        if need_old_logprobs:
            lay.old_logprobs = _f32(data_pack["packed_logprobs"], dev)
        if need_advantages:
            lay.advantages = _f32(data_pack["packed_advantages"], dev)
        if need_ref_logprobs and "packed_ref_logprobs" in data_pack:
            lay.ref_logprobs = _f32(data_pack["packed_ref_logprobs"], dev)
        return lay
    mask = _f32(~data_pack["prompt_mask"][:, 1:], dev)
    if "loss_mask" in data_pack:
        mask = mask * _f32(data_pack["loss_mask"][:, 1:], dev)
    lay = ResponseLayout(packed=False, response_mask=mask, valid_count=mask.sum().clamp(min=1),
                         response_len=mask.sum(dim=-1).clamp(min=1))
    if need_old_logprobs:
        lay.old_logprobs = _f32(data_pack["logprobs"][:, 1:], dev)
    if need_advantages:
        lay.advantages = _f32(data_pack["advantages"][:, 1:], dev)
    if need_ref_logprobs and "ref_logprobs" in data_pack:
        lay.ref_logprobs = _f32(data_pack["ref_logprobs"][:, 1:], dev)
    return lay


def sequence_sum(values: torch.Tensor, layout: ResponseLayout) -> torch.Tensor:
    """Sum of the masked values of every sequence -> ``[num_sequences]``."""
    masked = values * layout.response_mask.to(values.dtype)
    if not layout.packed:
        return masked.sum(dim=-1)
    if layout.seq_ids is None or layout.num_sequences is None:
        raise ValueError("packed sequence_sum requires seq_ids and num_sequences")
    out = torch.zeros(layout.num_sequences, device=values.device, dtype=values.dtype)
    return out.scatter_add(0, layout.seq_ids, masked)


def masked_mean(values: torch.Tensor, layout: ResponseLayout) -> torch.Tensor:
    return (values * layout.response_mask.to(values.dtype)).sum() / layout.valid_count.to(values.dtype)
