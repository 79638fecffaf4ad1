"""The in-process cluster (one worker thread behind the command queue) with a scripted worker, on the CPU: synchronous
and asynchronous calls, concurrent rollout requests sharing one running batch, failures, time-outs and shutdown.
Behaviours follow the reference's ``tests/test_protocol_cpu.py``."""

from __future__ import annotations

import asyncio
import threading
import time

import pytest
import torch

from areno_b200.engine.cluster import InProcessCluster, WorkerError, make_cluster
from areno_b200.engine.config import EngineConfig
from areno_b200.engine.protocol import Command, Op, TrainPayload
from tests.helpers import tiny_config
from tests.test_worker_loop_cpu import ScriptedWorker, _rollout_cmd


def _cluster(worker=None):
    worker = worker or ScriptedWorker()
    worker.device = torch.device("cpu")
    return InProcessCluster(EngineConfig(model=tiny_config()), worker=worker), worker


def test_sync_calls_return_one_result_per_rank():
    cluster, worker = _cluster()
    try:
        assert cluster.call(Op.MODEL_INFO) == [{"model_type": "scripted"}]
        assert cluster.call(Op.TRAIN, TrainPayload([[{}]], 3)) == [[{"loss": 1.0}]]
        assert cluster.worker is worker and ("train", 1, 3) in worker.log
        out = cluster.call(Op.INFER_ROLLOUT, _rollout_cmd(0, [[1, 1], [2]]).payload)[0]
        assert out.tokens == [[0, 0], [1]] and out.prompt_indices == [0, 1]
    finally:
        cluster.close()


def test_concurrent_async_rollouts_share_one_batch_and_resolve_separately():
    cluster, worker = _cluster()

    async def run():
        jobs = [cluster.call_async(Op.INFER_ROLLOUT, _rollout_cmd(0, [[i + 1] * (i + 2)]).payload) for i in range(3)]
        return await asyncio.gather(*jobs)

    try:
        outs = asyncio.run(run())
        assert [len(o[0].tokens[0]) for o in outs] == [2, 3, 4]
        engines = [e for e in worker.log if isinstance(e, tuple) and e[0] == "engine"]
        assert 1 <= len(engines) <= 3 and worker.engine.steps <= 2 + 3 + 4
        assert asyncio.run(cluster.call_async(Op.MODEL_INFO)) == [{"model_type": "scripted"}]
    finally:
        cluster.close()


def test_worker_failures_surface_with_the_remote_traceback():
    cluster, worker = _cluster()
    worker.model_info = lambda: (_ for _ in ()).throw(KeyError("no such model"))
    try:
        with pytest.raises(WorkerError, match="KeyError: 'no such model'"):
            cluster.call(Op.MODEL_INFO)
        with pytest.raises(WorkerError, match="worker failed in Op.MODEL_INFO"):
            asyncio.run(cluster.call_async(Op.MODEL_INFO))
        assert cluster.call(Op.PROBE_TRAIN_MEMORY) == [0.25]              # the worker lives on
    finally:
        cluster.close()


def test_calls_time_out_and_late_results_are_dropped():
    cluster, worker = _cluster()
    gate = threading.Event()
    worker.peak_memory_fraction = lambda: (gate.wait(5), 0.5)[1]
    try:
        t0 = time.time()
        with pytest.raises(TimeoutError, match="timed out"):
            cluster.call(Op.PROBE_TRAIN_MEMORY, timeout=0.3)
        assert time.time() - t0 < 3
        gate.set()
        assert cluster.call(Op.MODEL_INFO) == [{"model_type": "scripted"}]   # the late answer did not end up here
    finally:
        gate.set()
        cluster.close()


def test_close_is_idempotent_and_a_closed_cluster_refuses_calls():
    cluster, _ = _cluster()
    cluster.close()
    cluster.close()
    assert not cluster._thread.is_alive()
    with pytest.raises(WorkerError, match="closed"):
        cluster.call(Op.MODEL_INFO)
    with pytest.raises(WorkerError, match="closed"):
        asyncio.run(cluster.call_async(Op.MODEL_INFO))


def test_a_worker_thread_that_died_is_noticed():
    cluster, worker = _cluster()
    cluster._cmd_q.put(Command(Op.SHUTDOWN, 0))
    cluster._thread.join(5)
    with pytest.raises(WorkerError, match="exited without reporting"):
        cluster.call(Op.MODEL_INFO)
    cluster.close()


def test_layout_and_launcher_checks():
    with pytest.raises(ValueError, match="world_size == 1"):
        InProcessCluster(EngineConfig(model=tiny_config(), tp_size=1, dp_size=2))
    with pytest.raises(ValueError):
        make_cluster(EngineConfig(model=tiny_config()), launcher="carrier-pigeon")
