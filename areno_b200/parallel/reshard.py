"""Weight hand-off from the training layout to the rollout layout.

When training runs as pure data parallel every rank holds the complete bf16 parameters after the
post-step all-gather, so moving to a tensor-parallel rollout layout needs no communication at all:
each rank cuts its own shard out of its own replica.  ``reshard_into`` does that with the same
``tp_shard`` annotations the checkpoint code uses (row blocks for column-parallel weights, column
blocks for row-parallel ones, per-part blocks for merged projections, head blocks with KV
replication for fused QKV, padded row blocks for vocabulary-parallel tables).  The copies are plain
strided device copies (a few GB at HBM speed); nothing crosses NVLink.

The reference keeps one TP layout for both phases and therefore has no counterpart of this step;
its closest relative is the shard slicing in ``areno/engine/checkpoints/common.py`` used at load.
"""

from __future__ import annotations

import torch


def shard_of(full: torch.Tensor, like: torch.Tensor, shard, tp_rank: int, tp_size: int) -> list[tuple]:
    """Describe the local shard as ``[(dst_row_lo, dst_row_hi, src_view), ...]`` over views of
    ``full`` (the tp=1 parameter) for a local parameter shaped like ``like``."""
    kind, meta = shard if shard else (None, None)
    r = tp_rank
    if kind is None or tp_size == 1:
        return [(0, like.shape[0], full)]
    if kind == "col":
        n = like.shape[0]
        return [(0, n, full[r * n:(r + 1) * n])]
    if kind == "row":
        if meta is not None:   # uneven head layout: (first real input feature, real features); the rest stays zero
            lo, n = meta
            return [(0, like.shape[0], full[:, lo:lo + n], n)]
        n = like.shape[1]
        return [(0, like.shape[0], full[:, r * n:(r + 1) * n])]
    if kind == "vocab":
        per, valid = like.shape[0], int(meta)
        lo, hi = min(r * per, valid), min((r + 1) * per, valid)
        return [(0, hi - lo, full[lo:hi])] if hi > lo else []
    if kind == "merged":
        out, dst, src = [], 0, 0
        for n in meta:  # local rows of each fused part; the full part is tp_size times as tall
            out.append((dst, dst + n, full[src + r * n: src + (r + 1) * n]))
            dst += n
            src += n * tp_size
        return out
    if kind == "qkv":
        hq_rows, hkv, d, rep = meta[:4]  # local q rows (heads x q_mult), local kv heads, head_dim, kv replication
        q_rows, kv_rows = hq_rows * d, hkv * d
        q_full = q_rows * tp_size
        kv_full = kv_rows * (tp_size // rep)
        kv_rank = r // rep
        q_piece = (0, q_rows, full[r * q_rows:(r + 1) * q_rows])
        if len(meta) > 4:      # uneven head layout: real q rows [q_lo, q_lo + q_n) of q_all, local padding rows stay zero
            q_lo, q_n, q_all = (int(x) * d for x in meta[4:7])
            q_full = q_all
            q_piece = (0, q_n, full[q_lo:q_lo + q_n])
        return [
            q_piece,
            (q_rows, q_rows + kv_rows, full[q_full + kv_rank * kv_rows: q_full + (kv_rank + 1) * kv_rows]),
            (q_rows + kv_rows, q_rows + 2 * kv_rows,
             full[q_full + kv_full + kv_rank * kv_rows: q_full + kv_full + (kv_rank + 1) * kv_rows]),
        ]
    raise ValueError(f"unknown tp_shard kind {kind!r}")


@torch.no_grad()
def reshard_into(dst_model: torch.nn.Module, src_model: torch.nn.Module, tp_rank: int, tp_size: int) -> int:
    """Fill every parameter of ``dst_model`` (built in a ``tp_size``-wide layout) from ``src_model``
    (the same architecture at tp=1).  Returns the number of bytes written."""
    src = dict(src_model.named_parameters())
    written = 0
    seen: set[int] = set()
    for name, p in dst_model.named_parameters():
        if id(p) in seen:  # tied weights appear once
            continue
        seen.add(id(p))
        full = src.get(name)
        if full is None:
            raise KeyError(f"rollout parameter {name} has no training counterpart")
        shard = getattr(p, "tp_shard", None)
        pieces = shard_of(full.data, p.data, shard, tp_rank, tp_size)
        uneven = bool(shard) and ((shard[0] == "qkv" and len(shard[1]) > 4) or (shard[0] == "row" and shard[1] is not None))
        if uneven:
            p.data.zero_()            # padding heads: rows / columns that no piece covers must be zero
        covered = 0
        for piece in pieces:
            lo, hi, view = piece[:3]
            if len(piece) > 3:        # column-limited piece (row-parallel weight behind padded heads)
                p.data[lo:hi, : piece[3]].copy_(view)
            else:
                p.data[lo:hi].copy_(view)
            covered += hi - lo
        if covered < p.shape[0] and not uneven:
            p.data[covered:].zero_()  # vocabulary padding rows
        written += p.numel() * p.element_size()
    return written
