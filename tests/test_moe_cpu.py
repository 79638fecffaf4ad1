"""MoE on CPU (reference ops): plan invariants, block output against a dense per-token evaluation,
checkpoint round trip through the per-expert HF layout, and a generate + train step."""

from __future__ import annotations

import torch

from areno_b200.ops import moe as moe_ops
from areno_b200.parallel.context import single_process_context

from .helpers import tiny_config


def moe_config(**kw):
    base = dict(model_type="qwen3_moe", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, qk_norm=True,
                qkv_bias=False, norm_topk_prob=True)
    base.update(kw)
    return tiny_config(**base)


def test_plan_invariants():
    g = torch.Generator().manual_seed(0)
    ids = torch.stack([torch.randperm(8, generator=g)[:2] for _ in range(50)]).to(torch.int32)
    plan = moe_ops.align(ids, 0, 8)
    assert plan.max_rows % 128 == 0 and int(plan.counts.sum()) == 100
    er = plan.expert_rows.view(8, 2)
    assert all(int(o) % 128 == 0 and int(n) % 128 == 0 for o, n in er.tolist())
    rr, ro = plan.row_route, plan.route_row
    for route in range(100):
        assert int(rr[int(ro[route])]) == route
    # rows of one expert keep token order
    for e in range(8):
        lo, n = er[e].tolist()
        rows = rr[lo:lo + n]
        rows = rows[rows >= 0]
        assert torch.equal(rows, rows.sort().values)
        assert all(int(ids.reshape(-1)[r]) == e for r in rows.tolist())
    # a rank that owns experts 4..7 drops the other routes
    half = moe_ops.align(ids, 4, 4)
    assert int(half.counts.sum()) == int((ids >= 4).sum())
    assert torch.equal(half.route_row >= 0, (ids.reshape(-1) >= 4))


def test_block_matches_per_token_evaluation():
    from areno_b200.models.dense import init_weights
    from areno_b200.models.moe import SparseMoeBlock

    single_process_context()
    cfg = moe_config()
    block = SparseMoeBlock(cfg, torch.float32, "cpu")
    init_weights(block, 3)
    x = torch.randn(37, cfg.hidden_size)
    out = block(x)
    w, ids = block.router(x)
    ref = torch.zeros_like(x)
    inter = cfg.moe_intermediate_size
    for t in range(x.shape[0]):
        for j in range(cfg.num_experts_per_tok):
            e = int(ids[t, j])
            gu = block.experts.gate_up[e] @ x[t]
            a = torch.nn.functional.silu(gu[:inter]) * gu[inter:]
            ref[t] += w[t, j] * (block.experts.down[e] @ a)
    assert torch.allclose(out, ref, atol=1e-5)
    assert torch.allclose(w.sum(-1), torch.ones(37), atol=1e-6)


def test_checkpoint_round_trip_and_engine_step(tmp_path):
    from areno_b200.api import loss_fns
    from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig
    from areno_b200.engine.inference import SamplingParams
    from areno_b200.engine.worker import RankWorker
    from areno_b200.models import registry

    single_process_context()
    cfg = moe_config()
    adapter = registry.get_adapter("qwen3_moe")
    model = adapter.build(cfg)
    adapter.init_random(model, 1)
    path = str(tmp_path / "moe")
    adapter.save_weights(model, path, cfg)
    found, cfg2 = registry.config_from_pretrained(path)
    assert found.name == "qwen3_moe" and cfg2.num_experts == 8 and cfg2.moe_intermediate_size == 64
    cfg2.dtype = torch.float32
    model2 = adapter.build(cfg2)
    adapter.load_weights(model2, path, cfg2)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), model2.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2), n1

    ec = EngineConfig(model=cfg2, model_path=path, optimizer=OptimizerConfig(lr=1e-2, weight_decay=0.0),
                      runtime=RuntimeConfig(eager_decode=True, max_model_len=128, activation_checkpointing=False),
                      max_running_seqs=4)
    worker = RankWorker(ec, "cpu")
    worker.loss_fn = loss_fns.grpo_loss_fn
    prompts = [list(range(5, 20)), list(range(30, 41))]
    out = worker.rollout(prompts, SamplingParams(temperature=0.0), (), 5)
    assert [len(t) for t in out.tokens] == [5, 5]
    packs = []
    for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
        n = len(p) + len(toks)
        pm = torch.ones((1, n), dtype=torch.bool)
        pm[0, len(p):] = False
        lp = torch.zeros((1, n))
        lp[0, len(p):] = torch.tensor(lps)
        adv = torch.zeros((1, n))
        adv[0, len(p):] = 1.0
        packs.append(dict(input_ids=torch.tensor([p + toks]), lengths=torch.tensor([n]), prompt_mask=pm, logprobs=lp,
                          advantages=adv))
    before = worker.model.layers[0].mlp.experts.gate_up.detach().clone()
    gate_before = worker.model.layers[0].mlp.router.weight.detach().clone()
    stats = worker.train(packs)
    assert stats[-1]["stepped"] and stats[-1]["metrics"]["grad_norm"] > 0
    assert not torch.equal(before, worker.model.layers[0].mlp.experts.gate_up)
    assert not torch.equal(gate_before, worker.model.layers[0].mlp.router.weight)
