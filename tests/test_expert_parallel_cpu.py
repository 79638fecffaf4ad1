"""Two gloo ranks on CPU: a mixture-of-experts model with its experts dealt out over the data-parallel ranks
(expert parallelism through the collective fallback of ``parallel/ep.py``) must reproduce a single process that
holds all experts: same rollout tokens, same log-probs, same parameters after an optimizer step (shared
parameters on every rank, each rank's experts equal to the matching slice), and a checkpoint written by the
two ranks must load back into one process."""

from __future__ import annotations

import os
import socket
import tempfile
import traceback

import torch
import torch.multiprocessing as mp

from .helpers import tiny_config


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _moe_config():
    return tiny_config(model_type="qwen3_moe", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                       qk_norm=True, qkv_bias=False, norm_topk_prob=True)


def _prompts():
    g = torch.Generator().manual_seed(11)
    return [torch.randint(3, 512, (n,), generator=g).tolist() for n in (17, 30, 9, 24, 12)]


def _packs(prompts, outs):
    packs = []
    for p, toks, lps in zip(prompts, outs.tokens, outs.logprobs):
        n = len(p) + len(toks)
        pmask = torch.ones((1, n), dtype=torch.bool)
        pmask[0, len(p):] = False
        lp = torch.zeros((1, n))
        lp[0, len(p):] = torch.tensor(lps)
        adv = torch.zeros((1, n))
        adv[0, len(p):] = 1.0 if len(p) % 2 else -0.5
        packs.append(dict(input_ids=torch.tensor([p + toks]), lengths=torch.tensor([n]), prompt_mask=pmask, logprobs=lp,
                          advantages=adv))
    return packs


def _worker(cfg_kw):
    from areno_b200.api import loss_fns
    from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig
    from areno_b200.engine.worker import RankWorker

    cfg = EngineConfig(model=_moe_config(), model_path="", dummy_load=True, seed=3,
                       optimizer=OptimizerConfig(lr=1e-2, grad_clip_norm=1.0, weight_decay=0.0),
                       runtime=RuntimeConfig(eager_decode=True, max_model_len=128, activation_checkpointing=False),
                       max_running_seqs=8, **cfg_kw)
    w = RankWorker(cfg, "cpu")
    w.loss_fn = loss_fns.grpo_loss_fn
    return w


def _named(worker):
    return {n: p.detach().clone().float() for n, p in worker.model.named_parameters()}


def _rank_main(rank, world, port, ckpt_dir, ret):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        from areno_b200.engine.inference import SamplingParams
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        ctx = init_parallel(rank, world, tp_size=1, master_port=port, backend="gloo", device=torch.device("cpu"),
                            expert_parallel=True, timeout_s=120)
        assert ctx.ep_size == 2 and ctx.ep_rank == rank
        worker = _worker(dict(tp_size=1, dp_size=2, expert_parallel=True))
        ex = worker.model.layers[0].mlp.experts
        assert ex.ep and ex.e_local == 4 and ex.e_lo == 4 * rank and ctx.ep_runtime.impl == "collective"
        prompts = _prompts()
        mine = prompts[:3] if rank == 0 else prompts[3:]          # uneven on purpose: 3 and 2 prompts
        params = SamplingParams(temperature=0.0)
        first = worker.rollout(mine, params, (), 6)
        own = _packs(mine, first)
        n_mb = 3                                                   # rank 1 pads its two packs with an empty shard
        packs = [[(own[i] if i < len(own) else own[-1]) if r == rank else None for r in range(world)] for i in range(n_mb)]
        before = _named(worker)
        stats = worker.train(packs)
        after = _named(worker)
        rm = worker.role_manager()
        rm.score_token_budget = 40           # rank 0 scores in more micro-batches than rank 1: idle rounds on rank 1
        scored = rm.score_logprobs("actor", [p + t for p, t in zip(mine, first.tokens)], 0, 1)
        second = worker.rollout(mine, params, (), 6)
        # a rank without any prompt still takes part in the others' forward passes
        lonely = worker.rollout(mine[:1] if rank == 0 else [], params, (), 4)
        assert len(lonely.tokens) == (1 if rank == 0 else 0)
        worker.save_checkpoint(ckpt_dir)
        # resume: a checkpoint with the optimizer side-car, one more step, against a fresh pair of workers that load it
        os.environ["ARENO_SAVE_OPTIMIZER"] = "1"
        resume_dir = os.path.join(ckpt_dir, "resume")
        worker.save_checkpoint(resume_dir)
        os.environ.pop("ARENO_SAVE_OPTIMIZER")
        worker.train(packs)
        continued = _named(worker)
        from areno_b200.api import loss_fns
        from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig
        from areno_b200.engine.worker import RankWorker

        fresh = RankWorker(EngineConfig(model=_moe_config(), model_path=resume_dir, seed=99, tp_size=1, dp_size=2,
                                        expert_parallel=True,
                                        optimizer=OptimizerConfig(lr=1e-2, grad_clip_norm=1.0, weight_decay=0.0),
                                        runtime=RuntimeConfig(eager_decode=True, max_model_len=128,
                                                              activation_checkpointing=False), max_running_seqs=8), "cpu")
        fresh.loss_fn = loss_fns.grpo_loss_fn
        fresh.train(packs)
        assert fresh.trainer.global_step == worker.trainer.global_step == 2
        resumed = _named(fresh)
        for n, t in continued.items():
            assert (t - resumed[n]).abs().max() < 2e-6, (n, float((t - resumed[n]).abs().max()))
        # ranks that bring different numbers of micro-batches fail together with a message, instead of one of them
        # waiting for ever inside a token exchange
        try:
            worker.train(packs[: (2 if rank == 0 else 3)])
            uneven = "no error"
        except ValueError as exc:
            uneven = str(exc)
        assert "same number of micro-batches" in uneven and "between 2 and 3" in uneven, uneven
        ret[rank] = dict(first=first.tokens, first_lp=first.logprobs, second=second.tokens, before=before, after=after,
                         loss=[s["loss"] for s in stats], scored=scored,
                         local_buckets=sum(1 for b in worker.trainer.optimizer.buckets if b.local))
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


def test_expert_parallel_matches_a_single_process_with_all_experts():
    from areno_b200.engine.inference import SamplingParams
    from areno_b200.parallel.context import single_process_context

    port = _free_port()
    ret = mp.Manager().dict()
    with tempfile.TemporaryDirectory() as ckpt:
        mp.spawn(_rank_main, args=(2, port, ckpt, ret), nprocs=2, join=True)
        for r in range(2):
            assert isinstance(ret[r], dict), ret[r]
        assert ret[0]["local_buckets"] >= 1

        single_process_context()
        worker = _worker({})
        prompts = _prompts()
        params = SamplingParams(temperature=0.0)
        # same initial weights whatever the layout: shared parameters equal, experts equal slice by slice
        ref_before = _named(worker)
        for r in range(2):
            for n, t in ret[r]["before"].items():
                full = ref_before[n]
                want = full[4 * r:4 * r + 4] if ".experts." in n else full
                assert torch.equal(t, want), n
        first = worker.rollout(prompts, params, (), 6)
        assert ret[0]["first"] + ret[1]["first"] == first.tokens
        for a, b in zip(ret[0]["first_lp"] + ret[1]["first_lp"], first.logprobs):
            assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=1e-4)
        all_packs = _packs(prompts, first)
        # rank 0 trained packs 0, 1, 2 and rank 1 packs 3, 4, 4 in three micro-batches of two shards each; the
        # data-parallel average over two ranks of a sum over three micro-batches is six packs at half weight
        order = [all_packs[0], all_packs[3], all_packs[1], all_packs[4], all_packs[2], all_packs[4]]
        worker.train([[pk] for pk in order], gradient_accumulation_steps=6)
        ref_after = _named(worker)
        for r in range(2):
            for n, t in ret[r]["after"].items():
                full = ref_after[n]
                want = full[4 * r:4 * r + 4] if ".experts." in n else full
                assert (t - want).abs().max() < 3e-5, (n, float((t - want).abs().max()))
        assert any((ret[0]["after"][n] - ret[0]["before"][n]).abs().max() > 1e-4 for n in ret[0]["after"] if ".experts." in n)
        second = worker.rollout(prompts, params, (), 6)
        assert ret[0]["second"] + ret[1]["second"] == second.tokens
        scored = worker.role_manager().score_logprobs("actor", [p + t for p, t in zip(prompts, first.tokens)], 0, 1)
        for a, b in zip(ret[0]["scored"] + ret[1]["scored"], scored):
            assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=2e-4)
        # the two ranks' checkpoint (dense part + one expert file per rank) loads into one process
        from areno_b200.engine.config import EngineConfig, RuntimeConfig
        from areno_b200.engine.worker import RankWorker

        loaded = RankWorker(EngineConfig(model=_moe_config(), model_path=ckpt, runtime=RuntimeConfig(eager_decode=True, max_model_len=128)), "cpu")
        for n, p in loaded.model.named_parameters():
            assert (p.detach().float() - ref_after[n]).abs().max() < 3e-5, n


def test_runtime_picks_communicators_by_power_of_two_bucket_and_honours_a_pinned_size():
    from types import SimpleNamespace

    from areno_b200.parallel.ep import EpCommCollective, EpRuntime

    ctx = SimpleNamespace(ep_group=None, ep_size=4, ep_rank=1, ep_ctl_group=None)
    rt = EpRuntime(ctx, hidden=64, k=2, num_experts=8, device="cpu")
    assert rt.impl == "collective"                        # no CUDA device: library collectives
    assert [EpRuntime.bucket(n) for n in (0, 1, 64, 65, 4096, 4097)] == [64, 64, 64, 128, 4096, 8192]
    a, b = rt.comm(10), rt.comm(60)
    assert a is b and isinstance(a, EpCommCollective) and a.cap == 64 and (a.e_lo, a.e_local) == (2, 2)
    assert rt.comm(100).cap == 128 and len(rt._comms) == 2
    with rt.pinned(3000):                                 # the group-wide maximum decides, not the local size
        big = rt.comm(5)
        assert big.cap == 4096
        with rt.pinned(70):
            assert rt.comm(5).cap == 128
        assert rt.comm(1) is big
        try:
            rt.comm(5000)
        except ValueError as exc:
            assert "exceed" in str(exc)
        else:
            raise AssertionError("a pass larger than its pinned bucket must be refused")
    assert rt.comm(5).cap == 64 and rt.dropped() == 0
    rt.close()
    assert not rt._comms
