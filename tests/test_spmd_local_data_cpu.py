"""Two gloo ranks launched the SPMD way (every rank is its own driver process with RANK / WORLD_SIZE set): the
``Trainer`` in rank-local data mode (each rank passes only its own prompts and sequences, nothing is exchanged on
the host) must generate the same tokens and end at the same parameters as the default mode, in which every rank
passes the whole job's batch and the per-rank results are gathered."""

from __future__ import annotations

import os
import socket
import traceback

import torch
import torch.multiprocessing as mp

from .helpers import tiny_config


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _prompts():
    g = torch.Generator().manual_seed(21)
    return [torch.randint(3, 512, (n,), generator=g).tolist() for n in (11, 19, 8, 14)]


def _rank_main(rank, world, port, local, ret):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        from areno_b200.api import SamplingParams, Trainer, TrainSequence, grpo_loss_fn
        from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig
        from areno_b200.engine.worker import RankWorker
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        init_parallel(rank, world, tp_size=1, master_port=port, backend="gloo", device=torch.device("cpu"), timeout_s=120)
        cfg = EngineConfig(model=tiny_config(), dummy_load=True, seed=3, tp_size=1, dp_size=world, backend="gloo",
                           optimizer=OptimizerConfig(lr=1e-2, grad_clip_norm=1.0, weight_decay=0.0),
                           runtime=RuntimeConfig(eager_decode=True, max_model_len=128, activation_checkpointing=False),
                           max_running_seqs=8)
        worker = RankWorker(cfg, "cpu")
        trainer = Trainer.from_worker(worker, world_size=world, eos_ids=(0,), local_data=local)
        every = _prompts()
        # the default mode deals prompt i to rank i % world; the local mode is handed exactly that share
        mine = every[rank::world]
        params = SamplingParams(temperature=0.0, max_new_tokens=5, ignore_eos=True)
        with trainer.rollout_session(sampling_params=params):
            results = trainer.rollout_token_batch(mine if local else every, 1, params)
        if not local:
            results = results[rank::world]
        assert len(results) == len(mine)
        batch = []
        for p, res in zip(mine, results):
            seq = res.sequences[0]
            n = len(seq.resp_tokens)
            batch.append(TrainSequence(prompt_mask=[True] * len(p) + [False] * n, tokens=p + seq.resp_tokens,
                                       logprobs=[0.0] * len(p) + seq.resp_logprobs,
                                       advantages=[0.0] * len(p) + [0.5 if len(p) % 2 else -1.0] * n, eos_token_id=0))
        if local:
            stats = trainer.train(batch, grpo_loss_fn, mini_bs=1)
        else:
            # rebuild the whole job's batch in prompt order from every rank's sequences (they are deterministic:
            # greedy decoding), which the strided split of a 2-sequence micro-batch deals out as above
            import torch.distributed as dist

            parts = [None] * world
            dist.all_gather_object(parts, batch)
            whole = [parts[i % world][i // world] for i in range(len(every))]
            stats = trainer.train(whole, grpo_loss_fn, mini_bs=world)
        flat = torch.cat([p.detach().reshape(-1).float() for _n, p in sorted(worker.model.named_parameters())])
        ret[rank] = dict(tokens=[r.sequences[0].resp_tokens for r in results], flat=flat, loss=float(stats["loss"]))
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


def _run(local: bool):
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(2, _free_port(), local, ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], dict), ret[r]
    return [dict(ret[r]) for r in range(2)]


def test_rank_local_sdk_calls_match_the_gathered_mode():
    gathered, local = _run(False), _run(True)
    for r in range(2):
        assert local[r]["tokens"] == gathered[r]["tokens"]
        assert torch.equal(local[0]["flat"], local[1]["flat"])                    # data-parallel ranks stay in sync
        assert (local[r]["flat"] - gathered[r]["flat"]).abs().max() < 2e-6
    assert all(len(t) == 5 for t in local[0]["tokens"])
