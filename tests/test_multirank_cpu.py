"""Two gloo ranks on CPU: data-parallel training with a tensor-parallel rollout layout must reproduce
a single process (same tokens from rollout, same parameters after an optimizer step, and the
resharded rollout model must track the trained weights)."""

from __future__ import annotations

import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

from .helpers import tiny_config


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _prompts():
    g = torch.Generator().manual_seed(7)
    return [torch.randint(3, 512, (n,), generator=g).tolist() for n in (17, 30, 9, 24)]


def _packs(prompts, outs):
    packs = []
    for p, toks, lps in zip(prompts, outs.tokens, outs.logprobs):
        n = len(p) + len(toks)
        ids = torch.tensor([p + toks])
        pmask = torch.ones((1, n), dtype=torch.bool)
        pmask[0, len(p):] = False
        lp = torch.zeros((1, n))
        lp[0, len(p):] = torch.tensor(lps)
        adv = torch.zeros((1, n))
        adv[0, len(p):] = 1.0 if len(p) % 2 else -0.5
        packs.append(dict(input_ids=ids, lengths=torch.tensor([n]), prompt_mask=pmask, logprobs=lp, advantages=adv))
    return packs


def _worker(cfg_kw):
    from areno_b200.api import loss_fns
    from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig
    from areno_b200.engine.worker import RankWorker

    cfg = EngineConfig(model=tiny_config(), model_path="", dummy_load=True, seed=3,
                       optimizer=OptimizerConfig(lr=1e-2, grad_clip_norm=1.0, weight_decay=0.0),
                       runtime=RuntimeConfig(eager_decode=True, max_model_len=128, activation_checkpointing=False),
                       max_running_seqs=8, **cfg_kw)
    w = RankWorker(cfg, "cpu")
    w.loss_fn = loss_fns.grpo_loss_fn
    return w


def _scenario(worker, my_prompts, gather_tp, train_packs_of):
    from areno_b200.engine.inference import SamplingParams

    params = SamplingParams(temperature=0.0)
    first = worker.rollout(my_prompts, params, (), 6, gather_tp=gather_tp)
    stats = worker.train(train_packs_of(first))
    second = worker.rollout(my_prompts, params, (), 6, gather_tp=gather_tp)
    flat = torch.cat([p.detach().reshape(-1).float() for _n, p in sorted(worker.model.named_parameters())])
    return first, second, flat, stats


def _rank_main(rank, world, port, ret):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        ctx = init_parallel(rank, world, tp_size=1, master_port=port, backend="gloo", device=torch.device("cpu"),
                            rollout_tp_size=2, timeout_s=120)
        assert ctx.dp_size == 2 and ctx.rollout.tp_size == 2 and ctx.rollout.dp_size == 1
        worker = _worker(dict(tp_size=1, dp_size=2))
        assert worker.rollout_model is not worker.model
        prompts = _prompts()
        mine = prompts[rank * 2:(rank + 1) * 2]
        first, second, flat, stats = _scenario(worker, mine, True, lambda out: [[pk] for pk in _packs(mine, out)][:0] or
                                               _dp_packs(rank, world, prompts, mine, out))
        ret[rank] = dict(first=first.tokens, first_lp=first.logprobs, second=second.tokens, flat=flat,
                         loss=[s["loss"] for s in stats])
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


def _dp_packs(rank, world, prompts, mine, out):
    """Each micro-batch is a list with one shard per DP rank; a rank only fills in its own shard."""
    own = _packs(mine, out)
    return [[pk if r == rank else None for r in range(world)] for pk in own]


def test_dp_train_with_tp_rollout_matches_single_process():
    from areno_b200.parallel.context import single_process_context

    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], dict), ret[r]

    single_process_context()
    worker = _worker({})
    prompts = _prompts()

    def single_packs(out):
        packs = _packs(prompts, out)
        # two DP ranks x two micro-batches each, averaged == four micro-batches accumulated in the
        # order (rank0 mb0, rank1 mb0, rank0 mb1, rank1 mb1); order does not matter for the sum
        return [packs[0], packs[2], packs[1], packs[3]]

    first, second, flat, _ = _scenario(worker, prompts, False, single_packs)
    both_first = ret[0]["first"] + ret[1]["first"]
    assert both_first == first.tokens
    for a, b in zip(ret[0]["first_lp"] + ret[1]["first_lp"], first.logprobs):
        assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=1e-4)
    # both DP ranks hold identical parameters after the step, equal to the single-process result
    assert torch.allclose(ret[0]["flat"], ret[1]["flat"], atol=0, rtol=0)
    assert torch.allclose(ret[0]["flat"], flat, atol=2e-5)
    assert (ret[0]["flat"] - flat).abs().max() < 2e-5
    # the TP rollout after training used the resharded, updated weights
    assert ret[0]["second"] + ret[1]["second"] == second.tokens
    assert second.tokens != first.tokens


@pytest.mark.parametrize("tp,kv", [(2, 2), (4, 2)])
def test_reshard_matches_checkpoint_slicing(tp, kv):
    """Cutting shards out of a tp=1 model equals building the sharded model from the same seed-free
    source: logits of the TP model (summed over ranks by hand) match the full model."""
    from areno_b200.models.dense import DenseCausalLM, init_weights
    from areno_b200.parallel.context import ParallelContext, single_process_context, use_context
    from areno_b200.parallel.reshard import reshard_into

    single_process_context()
    cfg = tiny_config(num_attention_heads=4, num_key_value_heads=kv)
    full = DenseCausalLM(cfg)
    init_weights(full, 5)
    names = dict(full.named_parameters())
    for r in range(tp):
        with use_context(ParallelContext(rank=r, world_size=tp, tp_rank=r, tp_size=tp)):
            shard = DenseCausalLM(cfg)
        reshard_into(shard, full, r, tp)
        for name, p in shard.named_parameters():
            kind = (getattr(p, "tp_shard", None) or (None,))[0]
            f = names[name]
            if kind is None:
                assert torch.equal(p, f)
            elif kind == "col":
                n = p.shape[0]
                assert torch.equal(p, f[r * n:(r + 1) * n])
            elif kind == "row":
                n = p.shape[1]
                assert torch.equal(p, f[:, r * n:(r + 1) * n])
            elif kind == "qkv":
                hq, hkv, d, rep = p.tp_shard[1]
                assert torch.equal(p[: hq * d], f[r * hq * d:(r + 1) * hq * d])
                kr = r // rep
                q_full = hq * d * tp
                assert torch.equal(p[hq * d: hq * d + hkv * d], f[q_full + kr * hkv * d: q_full + (kr + 1) * hkv * d])
            elif kind == "merged":
                n0 = p.tp_shard[1][0]
                assert torch.equal(p[:n0], f[r * n0:(r + 1) * n0])
                assert torch.equal(p[n0:], f[n0 * tp + r * n0: n0 * tp + (r + 1) * n0])
            elif kind == "vocab":
                per = p.shape[0]
                lo, hi = min(r * per, 512), min((r + 1) * per, 512)
                assert torch.equal(p[: hi - lo], f[lo:hi])


def test_split_heads_deals_query_heads_over_ranks_sharing_a_kv_head():
    from areno_b200.models.layers import split_heads

    # 28 query / 4 KV heads at tp 8: two ranks per KV head, 4 + 3 query heads, one padding head on the second
    got = [split_heads(28, 4, 8, r) for r in range(8)]
    assert [g[0] for g in got] == [4] * 8 and [g[3:] for g in got] == [(1, 2)] * 8
    assert [(g[1], g[2]) for g in got] == [(0, 4), (4, 3), (7, 4), (11, 3), (14, 4), (18, 3), (21, 4), (25, 3)]
    covered = sorted(h for g in got for h in range(g[1], g[1] + g[2]))
    assert covered == list(range(28))
    # even layouts are untouched
    assert split_heads(28, 4, 4, 3) == (7, 21, 7, 1, 1)
    assert split_heads(32, 8, 16, 5) == (2, 10, 2, 1, 2)


def _uneven_rank(rank, world, port, ret):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        from areno_b200.engine.inference import SamplingParams
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        init_parallel(rank, world, tp_size=1, master_port=port, backend="gloo", device=torch.device("cpu"),
                      rollout_tp_size=4, timeout_s=120)
        worker = _uneven_worker(dict(tp_size=1, dp_size=4, rollout_tp_size=4))
        a = worker.rollout_model.layers[0].attn
        assert (a.hq, a.hkv) == (2, 1) and a.qkv.q_n == (2 if rank % 2 == 0 else 1)
        out = worker.rollout(_prompts()[rank:rank + 1], SamplingParams(temperature=0.0), (), 6, gather_tp=True)
        ret[rank] = dict(tokens=out.tokens, lp=out.logprobs)
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


def _uneven_worker(cfg_kw):
    from areno_b200.engine.config import EngineConfig, RuntimeConfig
    from areno_b200.engine.worker import RankWorker

    cfg = EngineConfig(model=tiny_config(num_attention_heads=6, num_key_value_heads=2), model_path="", dummy_load=True,
                       seed=3, runtime=RuntimeConfig(eager_decode=True, max_model_len=128), max_running_seqs=8, **cfg_kw)
    return RankWorker(cfg, "cpu")


def test_rollout_layout_wider_than_the_query_heads_divide_matches_single_process():
    """6 query / 2 KV heads on a 4-wide rollout layout: ranks get 2 + 1 query heads per KV group, the short ranks a
    zero-weight padding head.  Greedy tokens and log-probs equal the single-process model; training layouts
    still refuse the shape."""
    from areno_b200.engine.config import EngineConfig
    from areno_b200.engine.inference import SamplingParams
    from areno_b200.parallel.context import single_process_context

    with pytest.raises(ValueError, match="divisible by tp_size"):
        EngineConfig(model=tiny_config(num_attention_heads=6, num_key_value_heads=2), tp_size=4, dp_size=1)
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_uneven_rank, args=(4, port, ret), nprocs=4, join=True)
    for r in range(4):
        assert isinstance(ret[r], dict), ret[r]
    single_process_context()
    worker = _uneven_worker({})
    ref = worker.rollout(_prompts(), SamplingParams(temperature=0.0), (), 6)
    assert [ret[r]["tokens"][0] for r in range(4)] == ref.tokens
    for r in range(4):
        assert torch.allclose(torch.tensor(ret[r]["lp"][0]), torch.tensor(ref.logprobs[r]), atol=1e-4)
