"""The sharded AdamW on the CPU beyond the single-bucket case: many small buckets, gradients accumulated over
micro-batches (autograd gradients folded into the fp32 buffers, and gradients written straight into them), 8-bit
moments against fp32 moments, state that moves off the device and back, and the state dictionary round trip."""

from __future__ import annotations

import pytest
import torch

from areno_b200.engine.config import OptimizerConfig
from areno_b200.engine.optim import ShardedAdamW
from areno_b200.models.dense import DenseCausalLM, init_weights
from areno_b200.parallel.context import single_process_context
from tests.helpers import tiny_config


def _pair(dtype=torch.float32, **ocfg):
    single_process_context()
    cfg = tiny_config(num_hidden_layers=2, dtype=dtype)
    model, twin = DenseCausalLM(cfg), DenseCausalLM(cfg)
    init_weights(model, 3)
    twin.load_state_dict(model.state_dict())
    base = dict(lr=1e-2, weight_decay=0.05, betas=(0.9, 0.95), eps=1e-8, grad_clip_norm=None)
    base.update(ocfg)
    return model, twin, ShardedAdamW(model, OptimizerConfig(**base))


def _grads(model, seed, scale=0.01):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(p.shape, generator=g) * scale for p in model.parameters()]


def _same(model, twin, atol=1e-6):
    for (n, a), (_, b) in zip(model.named_parameters(), twin.named_parameters()):
        assert torch.allclose(a, b, atol=atol, rtol=1e-5), n


def test_many_small_buckets_update_like_one_big_optimizer():
    model, twin, opt = _pair(fp32_master_bucket_numel=4096)
    assert len(opt.buckets) > 8
    # every parameter is a view into its bucket and keeps its values
    for p, q in zip(model.parameters(), twin.parameters()):
        assert torch.equal(p, q) and p.main_grad.shape == p.shape and p.main_grad.dtype == torch.float32
    ref = torch.optim.AdamW(twin.parameters(), lr=1e-2, weight_decay=0.05, betas=(0.9, 0.95), eps=1e-8)
    for step in range(3):
        for p, q, g in zip(model.parameters(), twin.parameters(), _grads(model, step)):
            p.grad, q.grad = g.clone(), g.clone()
        ref.step()
        ref.zero_grad()
        opt.step(lr=1e-2)
    _same(model, twin)
    assert all(float(b.grad_flat.abs().sum()) == 0.0 for b in opt.buckets)            # zeroed for the next step
    assert all(p.grad is None for p in model.parameters())


def test_gradients_accumulate_over_micro_batches_before_one_step():
    model, twin, opt = _pair()
    ref = torch.optim.AdamW(twin.parameters(), lr=1e-2, weight_decay=0.05, betas=(0.9, 0.95), eps=1e-8)
    g1, g2 = _grads(model, 1), _grads(model, 2)
    # first micro-batch through autograd-style ``.grad`` and a fold; the second written into ``main_grad`` directly,
    # as the GEMM's wgrad epilogue does (flagged so that the fold does not add a stale ``.grad`` on top)
    for p, g in zip(model.parameters(), g1):
        p.grad = g.clone()
    opt.fold_param_grads()
    assert all(p.grad is None for p in model.parameters())
    for p, g in zip(model.parameters(), g2):
        p.main_grad.add_(g)
        p.grad = torch.full_like(p, 123.0)
        p.grad_added_to_main_grad = True
    for q, a, b in zip(twin.parameters(), g1, g2):
        q.grad = a + b
    ref.step()
    norm = opt.step(lr=1e-2)
    want = torch.sqrt(sum((a + b).float().pow(2).sum() for a, b in zip(g1, g2)))
    assert float(norm) == pytest.approx(float(want), rel=1e-5)
    _same(model, twin)


def test_clip_coefficient_is_applied_inside_the_update():
    model, twin, opt = _pair(grad_clip_norm=0.01)
    ref = torch.optim.AdamW(twin.parameters(), lr=1e-2, weight_decay=0.05, betas=(0.9, 0.95), eps=1e-8)
    for p, q, g in zip(model.parameters(), twin.parameters(), _grads(model, 5, scale=1.0)):
        p.grad, q.grad = g.clone(), g.clone()
    torch.nn.utils.clip_grad_norm_(twin.parameters(), 0.01)
    ref.step()
    norm = opt.step(lr=1e-2)                     # clip from the config
    assert float(norm) > 1.0                     # the norm before clipping is what is reported
    _same(model, twin, atol=2e-6)


def test_eight_bit_moments_track_the_fp32_optimizer():
    model, twin, opt8 = _pair(dtype=torch.bfloat16, adam_8bit=True, weight_decay=0.0)      # fp32 parameters keep fp32 moments
    opt32 = ShardedAdamW(twin, OptimizerConfig(lr=1e-2, weight_decay=0.0, betas=(0.9, 0.95), eps=1e-8, grad_clip_norm=None))
    start = [p.detach().clone() for p in model.parameters()]
    for step in range(4):
        for p, q, g in zip(model.parameters(), twin.parameters(), _grads(model, 10 + step)):
            p.main_grad.add_(g)               # bf16 parameters: gradients arrive in the fp32 buffers
            q.main_grad.add_(g)
        opt8.step(lr=1e-2)
        opt32.step(lr=1e-2)
    b = opt8.buckets[0]
    assert b.m.dtype == torch.int8 and b.v.dtype == torch.uint8 and b.master is None and b.m_scale.numel() * 32 >= b.shard
    moved = torch.cat([(p.detach() - s).float().reshape(-1) for p, s in zip(model.parameters(), start)])
    moved32 = torch.cat([(q.detach() - s).float().reshape(-1) for q, s in zip(twin.parameters(), start)])
    # the quantised moments change individual updates a little; the step as a whole goes the same way
    cos = torch.nn.functional.cosine_similarity(moved, moved32, dim=0)
    assert float(cos) > 0.98 and float((moved - moved32).abs().max()) < 2.5e-2


def test_state_moves_to_the_host_and_back_and_round_trips_through_a_dictionary():
    model, twin, opt = _pair()
    other = ShardedAdamW(twin, OptimizerConfig(lr=1e-2, weight_decay=0.05, betas=(0.9, 0.95), eps=1e-8, grad_clip_norm=None))
    for p, g in zip(model.parameters(), _grads(model, 1)):
        p.grad = g.clone()
    opt.step(lr=1e-2)
    opt.offload_state()                           # on the CPU a no-op for placement; the bookkeeping must survive it
    opt.onload_state(torch.device("cpu"))
    state = opt.state_dict()
    assert state["step"] == 1 and state["dp_size"] == 1 and len(state["buckets"]) == len(opt.buckets)
    twin.load_state_dict(model.state_dict())
    other.load_state_dict(state)
    for p, q, g in zip(model.parameters(), twin.parameters(), _grads(model, 2)):
        p.grad, q.grad = g.clone(), g.clone()
    opt.step(lr=1e-2)
    other.step(lr=1e-2)
    assert other.step_count == 2
    _same(model, twin, atol=0.0)
    state["dp_size"] = 2
    with pytest.raises(ValueError, match="different sharding layout"):
        other.load_state_dict(state)


def test_frozen_parameters_are_left_out():
    single_process_context()
    model = DenseCausalLM(tiny_config(num_hidden_layers=1))
    init_weights(model, 3)
    frozen = model.embed.weight
    frozen.requires_grad_(False)
    before = frozen.detach().clone()
    opt = ShardedAdamW(model, OptimizerConfig(lr=1e-1, weight_decay=0.1))
    assert all(frozen is not p for b in opt.buckets for p in b.params) and not hasattr(frozen, "main_grad")
    for p in model.parameters():
        if p.requires_grad:
            p.grad = torch.ones_like(p)
    opt.step(lr=1e-1)
    assert torch.equal(frozen, before)
