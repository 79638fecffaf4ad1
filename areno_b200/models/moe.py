"""Sparse mixture-of-experts decoder (Qwen3-MoE family): softmax top-k router with fp32 gate, experts
sharded over the TP group (every rank sees all tokens and serves the routes that hit its experts,
then the partial outputs are summed over the group) or, with expert parallelism, over the data-parallel
group (tokens are exchanged with the experts' owners over peer memory and the outputs come back the same
way), grouped tcgen05 GEMMs over expert-sorted rows.

Structure of ``areno/models/qwen3/model.py:75-231`` in the reference; the per-expert cuBLAS loop,
the host sync for offsets and the Triton inference path are replaced by the device-side plan and
the grouped GEMM of ``ops/moe.py``, used for training and inference alike.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ..engine.config import ModelConfig
from ..ops import activation, moe as moe_ops
from ..parallel import collectives as coll
from ..parallel.context import get_context
from .dense import DecoderLayer, DenseCausalLM
from .layers import GatedMLP, _param


class TopKRouter(nn.Module):
    """``logits = x @ gate^T`` in fp32 (the gate is kept in fp32 and replicated over TP)."""

    def __init__(self, cfg: ModelConfig, device):
        super().__init__()
        self.k = cfg.num_experts_per_tok
        self.renorm = cfg.norm_topk_prob
        self.weight = _param((cfg.num_experts, cfg.hidden_size), torch.float32, device)
        self.weight.tp_replicated_grad = True

    def forward(self, x):
        return moe_ops.topk_softmax(moe_ops.router_logits(x, self.weight), self.k, self.renorm)


class Experts(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        ctx = get_context()
        e = cfg.num_experts
        # Expert parallelism: the experts are dealt out over the data-parallel group and the TOKENS travel to them
        # (parallel/ep.py); otherwise they are sharded over the TP group, whose ranks all see every token.
        self.ep = ctx.ep_size > 1
        ways, rank = (ctx.ep_size, ctx.ep_rank) if self.ep else (ctx.tp_size, ctx.tp_rank)
        assert e % ways == 0, "num_experts must be divisible by the size of the group that shards the experts"
        self.e_local = e // ways
        self.e_lo = rank * self.e_local
        self.inter = cfg.moe_intermediate_size
        self.act = cfg.hidden_act
        self.gate_up = _param((self.e_local, 2 * self.inter, cfg.hidden_size), dtype, device)
        self.down = _param((self.e_local, cfg.hidden_size, self.inter), dtype, device)
        self.gate_up.expert_range = (self.e_lo, e)      # read by the seeded random init
        self.down.expert_range = (self.e_lo, e)
        if self.ep:
            # every data-parallel rank owns different experts: the optimizer neither reduces nor gathers these
            self.gate_up.ep_local = True
            self.down.ep_local = True
            if ctx.ep_runtime is None:
                from ..parallel.ep import EpRuntime

                ctx.ep_runtime = EpRuntime(ctx, cfg.hidden_size, cfg.num_experts_per_tok, e, device)
        else:
            # dim-0 (expert) sharding: same slicing as a column-parallel weight
            self.gate_up.tp_shard = ("col", None)
            self.down.tp_shard = ("col", None)

    def _forward_ep(self, x, weights, ids):
        comm = get_context().ep_runtime.comm(x.shape[0])
        rows, plan = comm.dispatch(x, ids)
        gu = moe_ops.grouped_linear(rows, self.gate_up, plan.moe)
        act = activation.silu_and_mul if self.act == "silu" else activation.gelu_tanh_and_mul
        a = act(gu, plan.moe.row_route)
        ys = moe_ops.grouped_linear(a, self.down, plan.moe)
        return comm.combine(ys, weights, plan), plan.moe

    def forward(self, x, weights, ids):
        if self.ep:
            return self._forward_ep(x, weights, ids)
        plan = moe_ops.align(ids, self.e_lo, self.e_local)
        xs = moe_ops.permute(x, plan)
        gu = moe_ops.grouped_linear(xs, self.gate_up, plan)
        act = activation.silu_and_mul if self.act == "silu" else activation.gelu_tanh_and_mul
        a = act(gu, plan.row_route)
        ys = moe_ops.grouped_linear(a, self.down, plan)
        out = moe_ops.combine(ys, plan, weights)
        return coll.reduce_from_tp(out), plan


class SparseMoeBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.router = TopKRouter(cfg, device)
        self.experts = Experts(cfg, dtype, device)
        self.shared = None
        self.shared_gate = None
        if cfg.shared_expert_intermediate_size:
            self.shared = GatedMLP(cfg.hidden_size, cfg.shared_expert_intermediate_size, cfg.hidden_act, False, dtype,
                                   device)
            if (cfg.extra or {}).get("shared_expert_gate"):
                # per-token sigmoid gate on the shared expert's output (Qwen3.5-MoE)
                self.shared_gate = _param((cfg.hidden_size,), dtype, device)
                self.shared_gate.tp_replicated_grad = "same"
        self.last_counts = None  # tokens per local expert of the latest forward (device tensor, for metrics)

    def forward(self, x):
        # Router and routed experts see the token through copy_to_tp: each rank back-propagates only the routes of
        # its own experts (into the token and, through the routing weights, into the router), and the TP sum in
        # copy_to_tp's backward completes the token gradient.  The shared expert sums its own input gradient, and
        # its sigmoid gate is computed identically on every rank, so both read the token directly.
        x_tp = coll.copy_to_tp(x)
        weights, ids = self.router(x_tp)
        out, plan = self.experts(x_tp, weights, ids)
        self.last_counts = plan.counts
        if self.shared is not None:
            shared = self.shared(x)
            if self.shared_gate is not None:
                # under sequence parallelism `shared` holds this rank's rows only, `x` all of them
                shared = shared * coll.local_rows(torch.sigmoid(torch.nn.functional.linear(x, self.shared_gate.unsqueeze(0))))
            out = out + shared
        return out


def is_sparse_layer(cfg: ModelConfig, i: int) -> bool:
    if not cfg.num_experts:
        return False
    extra = cfg.extra or {}
    if i in set(extra.get("mlp_only_layers") or []):
        return False
    step = int(extra.get("decoder_sparse_step", 1) or 1)
    return (i + 1) % step == 0


class MoeCausalLM(DenseCausalLM):
    def _make_layer(self, i, dtype, device):
        cfg = self.cfg
        mlp = SparseMoeBlock(cfg, dtype, device) if is_sparse_layer(cfg, i) else None
        return DecoderLayer(cfg, i, dtype, device, mlp=mlp)

    def finalize_router_expert_bias(self, tp_group=None, dp_group=None) -> None:
        """Softmax routers carry no selection bias: nothing to update after a step."""
        return None

    @torch.no_grad()
    def ep_idle_forward(self) -> None:
        """Expert parallelism: take part in one forward pass of the OTHER ranks without tokens of one's own.  Every
        MoE layer still has to publish a routing table, serve the routes that hit the local experts and answer
        the exchange; attention and the dense parts have nothing to do.  One zero token with zero routing weights
        stands in for the batch."""
        cfg = self.cfg
        k = cfg.num_experts_per_tok
        x = w = ids = None
        for layer in self.layers:
            mlp = getattr(layer, "mlp", None)
            if isinstance(mlp, SparseMoeBlock) and mlp.experts.ep:
                if x is None:
                    ref = mlp.experts.gate_up
                    x = torch.zeros((1, cfg.hidden_size), dtype=ref.dtype, device=ref.device)
                    w = torch.zeros((1, k), dtype=torch.float32, device=ref.device)
                    ids = torch.arange(k, dtype=torch.int32, device=ref.device).unsqueeze(0)
                mlp.experts(x, w, ids)
