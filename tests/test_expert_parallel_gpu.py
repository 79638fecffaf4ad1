"""Two GPUs: a bf16 mixture-of-experts model trained and rolled out with expert parallelism.  The scenario (scoring,
a sampled rollout through the CUDA-graph decode path, one optimizer step, scoring again) runs once on the
peer-memory exchange kernels and once on the library-collective fallback; the two must agree to bf16 accuracy, no
route may be dropped and no bounded wait may have run out.  Skipped on a box with fewer than two GPUs."""

from __future__ import annotations

import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rows(rank: int):
    g = torch.Generator().manual_seed(100 + rank)
    return [torch.randint(3, 4000, (n,), generator=g).tolist() for n in ((70, 33, 51) if rank == 0 else (40, 90))]


def _packs(rank: int, world: int, rows):
    packs = []
    for i in range(3):                              # rank 1 has two rows: it repeats the last one
        r = rows[min(i, len(rows) - 1)]
        n = len(r)
        pmask = torch.ones((1, n), dtype=torch.bool)
        pmask[0, n // 2:] = False
        g = torch.Generator().manual_seed(7 * i + rank)
        pk = dict(input_ids=torch.tensor([r]), lengths=torch.tensor([n]), prompt_mask=pmask,
                  logprobs=-torch.rand((1, n), generator=g) - 7.0, advantages=torch.randn((1, n), generator=g))
        packs.append([pk if q == rank else None for q in range(world)])
    return packs


def _rank_main(rank, world, port, impl, ret):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        os.environ["ARENO_EP_IMPL"] = impl
        os.environ["ARENO_EP_WAIT_MS"] = "5000"
        from areno_b200.api import loss_fns
        from areno_b200.engine.config import EngineConfig, ModelConfig, OptimizerConfig, RuntimeConfig
        from areno_b200.engine.inference import SamplingParams
        from areno_b200.engine.worker import RankWorker
        from areno_b200.ops import _lib
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        ctx = init_parallel(rank, world, tp_size=1, master_port=port, device=dev, expert_parallel=True, timeout_s=120)
        mcfg = ModelConfig(model_type="qwen3_moe", vocab_size=4096, hidden_size=512, intermediate_size=1024,
                           num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                           qk_norm=True, qkv_bias=False, rope_theta=1e4, num_experts=16, num_experts_per_tok=4,
                           moe_intermediate_size=256, norm_topk_prob=True, max_position_embeddings=1024)
        cfg = EngineConfig(model=mcfg, dummy_load=True, seed=5, tp_size=1, dp_size=world, expert_parallel=True,
                           devices=list(range(world)),
                           optimizer=OptimizerConfig(lr=1e-3, grad_clip_norm=1.0, weight_decay=0.0),
                           runtime=RuntimeConfig(max_model_len=256, activation_checkpointing=False), max_running_seqs=8)
        worker = RankWorker(cfg, dev)
        worker.loss_fn = loss_fns.grpo_loss_fn
        assert ctx.ep_runtime.impl == impl
        rows = _rows(rank)
        scored = worker.role_manager().score_logprobs("actor", rows, 0, 1)
        out = worker.rollout([r[:20] for r in rows], SamplingParams(temperature=1.0, seed=9), (), 12)
        # a rank without prompts joins the other rank's prefill with an idle pass and its decode steps with no slot active
        lonely = worker.rollout([rows[0][:16]] if rank == 0 else [], SamplingParams(temperature=1.0, seed=3), (), 5)
        assert [len(t) for t in lonely.tokens] == ([5] if rank == 0 else [])
        graphs = len(worker.infer._graphs)                  # building the trainer re-points the weights and drops them
        stats = worker.train(_packs(rank, world, rows))
        scored2 = worker.role_manager().score_logprobs("actor", rows, 0, 1)
        torch.cuda.synchronize()
        _lib.check_status(dev)
        ret[rank] = dict(scored=scored, scored2=scored2, loss=[s["loss"] for s in stats],
                         lens=[len(t) for t in out.tokens], lp=out.logprobs, dropped=ctx.ep_runtime.dropped(),
                         graphs=graphs)
        ctx.ep_runtime.close()
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


def _run(impl: str):
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(2, _free_port(), impl, ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], dict), ret[r]
    return [dict(ret[r]) for r in range(2)]


def test_expert_parallel_peer_kernels_agree_with_the_collective_fallback():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    peer, coll = _run("peer"), _run("collective")
    for r in range(2):
        p, c = peer[r], coll[r]
        assert p["dropped"] == 0 and p["graphs"] >= 1           # the decode step ran from a captured graph
        assert p["lens"] == [12] * len(p["lens"]) == c["lens"]
        assert all(torch.isfinite(torch.tensor(x)).all() and max(x) <= 0.0 for x in p["lp"])
        for a, b in zip(p["scored"], c["scored"]):
            assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=5e-2), (max(abs(x - y) for x, y in zip(a, b)))
        for a, b in zip(p["loss"], c["loss"]):
            assert abs(a - b) < 5e-2 * max(1.0, abs(b))
        moved = max(abs(x - y) for a, b in zip(p["scored"], p["scored2"]) for x, y in zip(a, b))
        assert moved > 1e-3                                       # the step changed the model
        for a, b in zip(p["scored2"], c["scored2"]):
            assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=8e-2)
