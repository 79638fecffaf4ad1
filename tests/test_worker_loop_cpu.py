"""The rank worker's command loop against a scripted worker and engine, on the CPU: which worker method every command
reaches, how rollout requests join a running batch and come back one by one, what waits behind a command that cannot
join, cancellation, and how failures travel to the driver.  Behaviours follow the worker half of the reference's
``tests/test_inference_scheduler_cpu.py``."""

from __future__ import annotations

from types import SimpleNamespace

import pytest

from areno_b200.engine.inference import RolloutOutput, SamplingParams
from areno_b200.engine.protocol import (CachePayload, Command, Op, RolesPayload, RolloutPayload, SavePayload, ScorePayload,
                                        TrainPayload, TrainValuesPayload)
from areno_b200.engine.worker_loop import WorkerLoop, execute, make_queue_getter
from areno_b200.parallel.context import single_process_context


class ScriptedEngine:
    """Every request finishes after ``len(prompt)`` decode steps with tokens ``[rid] * steps``."""

    def __init__(self, max_model_len=64):
        self.max_model_len = max_model_len
        self._requests: dict[int, SimpleNamespace] = {}
        self.begun = None
        self.steps = 0
        self.cancelled = False

    def begin(self, params, eos, max_new):
        self.begun = (params, tuple(eos), max_new)

    def add_request(self, prompt, max_new, tag=None, stream=None):
        rid = len(self._requests)
        self._requests[rid] = SimpleNamespace(rid=rid, prompt=list(prompt), left=len(prompt), tag=tag, stream=stream,
                                              tokens=None, logprobs=None, reason="", done=False)
        return rid

    @property
    def idle(self):
        return all(r.done for r in self._requests.values())

    def step(self):
        self.steps += 1
        out = []
        for r in self._requests.values():
            if r.done:
                continue
            r.left -= 1
            if r.left <= 0:
                r.done, r.reason = True, "stop"
                r.tokens, r.logprobs = [r.rid] * len(r.prompt), [-1.0] * len(r.prompt)
                out.append(r)
        return out

    def cancel_all(self):
        self.cancelled = True
        for r in self._requests.values():
            if not r.done:
                r.done, r.tokens, r.logprobs = True, [], []


class ScriptedWorker:
    def __init__(self, tp=1, ep=1, dp_rank=0):
        self.rollout_ctx = SimpleNamespace(tp_size=tp, ep_size=ep, dp_rank=dp_rank)
        self.engine = ScriptedEngine()
        self.log: list = []
        self.infer = None

    def prepare_for_rollout(self):
        self.log.append("prepare_for_rollout")

    def prepare_actor_onloaded(self):
        self.log.append("onload")

    def prepare_for_train(self):
        self.log.append("prepare_for_train")

    def inference_engine(self, slots, need_len):
        self.log.append(("engine", slots, need_len))
        return self.engine

    def rollout(self, prompts, params, eos, max_new, max_running=None, progress_interval_s=None, stream_ids=None):
        self.log.append(("rollout", len(prompts), max_running))
        self.stream_ids = stream_ids
        return RolloutOutput(tokens=[[9] for _ in prompts], logprobs=[[0.0] for _ in prompts],
                             finish_reasons=["stop"] * len(prompts))

    def train(self, packs, accumulation):
        self.log.append(("train", len(packs), accumulation))
        return [{"loss": 1.0}]

    def role_manager(self):
        worker = self

        class Roles:
            def ensure_roles(self, roles):
                worker.log.append(("roles", sorted(roles)))

            def score_logprobs(self, role, rows, pad, micro):
                return [("lp", role, r, pad, micro) for r in rows]

            def score_values(self, role, rows, pad):
                return [("v", role, r, pad) for r in rows]

            def score_rewards(self, role, rows, pad):
                return [("r", role, r, pad) for r in rows]

            def train_values(self, role, packs, accumulation, cliprange_value, value_loss_coef):
                return {"role": role, "packs": len(packs), "clip": cliprange_value, "coef": value_loss_coef}

        return Roles()

    def save_checkpoint(self, path):
        self.log.append(("save", path))

    def probe_rollout_cache(self, slots, length):
        return 0.5

    def peak_memory_fraction(self):
        return 0.25

    def model_info(self):
        return {"model_type": "scripted"}


def _rollout_cmd(rid, prompts, indices=None, max_new=4, **params):
    indices = list(range(len(prompts))) if indices is None else indices
    return Command(Op.INFER_ROLLOUT, rid, RolloutPayload([prompts], [indices], max_new_tokens=max_new,
                                                         sampling_params=SamplingParams(**params), max_running_seqs=4))


def _loop(worker, commands):
    """Feed ``commands`` (a list, consumed in order; a callable entry is evaluated lazily) and collect results."""
    feed, results = list(commands), []

    def get_cmd(timeout):
        if not feed:
            if timeout is None:
                return Command(Op.SHUTDOWN, -1)
            return None
        head = feed[0]
        if callable(head):                       # hold the command back until the predicate says so
            ready, cmd = head()
            if not ready:
                if timeout is None:
                    raise AssertionError("the loop blocked on a command that is being held back")
                return None
            feed.pop(0)
            return cmd
        return feed.pop(0)

    loop = WorkerLoop(worker, rank=3, get_cmd=get_cmd, put_result=results.append)
    loop.run()
    return results


@pytest.fixture(autouse=True)
def _ctx():
    single_process_context()


# ------------------------------------------------------------------------------------------------ plain commands

def test_every_command_reaches_its_worker_method():
    w = ScriptedWorker()
    rows = [[[1, 2], [3]]]
    assert execute(w, Command(Op.TRAIN, 0, TrainPayload([[{}], [{}]], 2))) == [{"loss": 1.0}]
    assert execute(w, Command(Op.SCORE_LOGPROBS, 0, ScorePayload("ref", rows, 7, 4))) == [("lp", "ref", [1, 2], 7, 4),
                                                                                      ("lp", "ref", [3], 7, 4)]
    assert execute(w, Command(Op.SCORE_VALUES, 0, ScorePayload("critic", rows, 7)))[0] == ("v", "critic", [1, 2], 7)
    assert execute(w, Command(Op.SCORE_REWARDS, 0, ScorePayload("rm", rows, 7)))[1] == ("r", "rm", [3], 7)
    assert execute(w, Command(Op.TRAIN_VALUES, 0, TrainValuesPayload("critic", [[{}]], None, 0.3, 0.7))) == {
        "role": "critic", "packs": 1, "clip": 0.3, "coef": 0.7}
    assert execute(w, Command(Op.ENSURE_ROLES, 0, RolesPayload({"ref": 1, "critic": 2}))) is None
    assert execute(w, Command(Op.SAVE_CHECKPOINT, 0, SavePayload("/tmp/ck"))) == "/tmp/ck"
    assert execute(w, Command(Op.PROBE_ROLLOUT_CACHE, 0, CachePayload(4, 128))) == 0.5
    assert execute(w, Command(Op.PROBE_TRAIN_MEMORY, 0)) == 0.25
    assert execute(w, Command(Op.MODEL_INFO, 0)) == {"model_type": "scripted"}
    for op in (Op.ROLLOUT_SESSION_BEGIN, Op.ROLLOUT_SESSION_SYNC, Op.ROLLOUT_SESSION_END, Op.CANCEL):
        assert execute(w, Command(op, 0)) is None
    assert w.log == [("train", 2, 2), ("roles", ["critic", "ref"]), ("save", "/tmp/ck"), "onload", "prepare_for_train"]
    with pytest.raises(ValueError, match="unsupported op"):
        execute(w, Command(Op.SHUTDOWN, 0))


def test_blocking_rollout_answers_for_this_rows_prompts_only():
    w = ScriptedWorker(dp_rank=1)
    payload = RolloutPayload([[[1]], [[2], [3]]], [[0], [1, 2]], max_new_tokens=4, max_running_seqs=2)
    out = execute(w, Command(Op.INFER_ROLLOUT, 0, payload))
    assert out.prompt_indices == [1, 2] and out.tokens == [[9], [9]] and w.log == [("rollout", 2, 2)]
    assert w.stream_ids == [1, 2]            # seeded samples are numbered by their position in the whole request
    empty = RolloutPayload([[[1]], []], [[0], []], max_new_tokens=4)
    out = execute(w, Command(Op.INFER_ROLLOUT, 0, empty))
    assert out.prompt_indices == [] and out.tokens == [] and len(w.log) == 1           # no rollout was started


def test_a_rank_without_prompts_still_joins_under_expert_parallelism():
    w = ScriptedWorker(ep=2, dp_rank=1)
    execute(w, Command(Op.INFER_ROLLOUT, 0, RolloutPayload([[[1]], []], [[0], []], max_new_tokens=4)))
    assert w.log == [("rollout", 0, 64)]


# -------------------------------------------------------------------------------------------- continuous rollout

def test_a_single_request_runs_to_its_end():
    w = ScriptedWorker()
    results = _loop(w, [_rollout_cmd(5, [[1, 1, 1], [2]], indices=[4, 6])])
    assert [(r.rank, r.request_id, r.ok) for r in results] == [(3, 5, True), (3, -1, True)]
    out = results[0].payload
    assert out.prompt_indices == [4, 6] and out.tokens == [[0, 0, 0], [1]] and out.finish_reasons == ["stop", "stop"]
    assert w.engine.steps == 3 and w.log[0] == "prepare_for_rollout" and w.log[1] == ("engine", 4, 64)
    assert w.engine.begun[2] == 4 and [r.stream for r in w.engine._requests.values()] == [None, None]


def test_compatible_requests_join_the_running_batch_and_return_as_they_finish():
    w = ScriptedWorker()
    long_ = _rollout_cmd(1, [[1] * 5])
    short = _rollout_cmd(2, [[2]])
    mid = _rollout_cmd(3, [[3] * 3])
    results = _loop(w, [long_, short, mid])
    assert [r.request_id for r in results] == [2, 3, 1, -1]          # in order of completion, not of arrival
    assert w.engine.steps == 5                                       # one batch: the longest request sets the length
    assert results[0].payload.tokens == [[1]] and results[2].payload.tokens == [[0] * 5]
    assert sum(1 for e in w.log if isinstance(e, tuple) and e[0] == "engine") == 1


def test_a_request_arriving_mid_batch_is_admitted_between_steps():
    w = ScriptedWorker()
    late = _rollout_cmd(2, [[7, 7]])
    results = _loop(w, [_rollout_cmd(1, [[1] * 4]), lambda: (w.engine.steps >= 2, late)])
    assert [r.request_id for r in results] == [1, 2, -1] or [r.request_id for r in results] == [2, 1, -1]
    assert w.engine.steps == 4 and len(w.engine._requests) == 2
    by_id = {r.request_id: r.payload for r in results}
    assert by_id[2].tokens == [[1, 1]] and by_id[1].tokens == [[0] * 4]


def test_a_request_without_local_rows_is_acknowledged_at_once():
    w = ScriptedWorker()
    nothing_here = Command(Op.INFER_ROLLOUT, 8, RolloutPayload([[]], [[]], max_new_tokens=4, max_running_seqs=4))
    results = _loop(w, [_rollout_cmd(1, [[1, 1]]), nothing_here])
    assert [r.request_id for r in results] == [8, 1, -1]
    assert results[0].payload.prompt_indices == [] and results[0].payload.tokens == []


def test_other_commands_wait_for_the_batch_and_keep_their_order():
    w = ScriptedWorker()
    train = Command(Op.TRAIN, 20, TrainPayload([[{}]], None))
    behind = _rollout_cmd(30, [[5]])
    results = _loop(w, [_rollout_cmd(10, [[1] * 3]), train, behind])
    assert [r.request_id for r in results] == [10, 20, 30, -1]
    assert results[1].payload == [{"loss": 1.0}]
    # the request behind the training command did not slip into the first batch: it got a batch of its own
    assert sum(1 for e in w.log if isinstance(e, tuple) and e[0] == "engine") == 2
    assert w.log.index(("train", 1, None)) < [i for i, e in enumerate(w.log) if e == "prepare_for_rollout"][1]


def test_requests_with_other_sampling_or_too_long_for_the_engine_wait_for_their_own_batch():
    w = ScriptedWorker()
    hot = _rollout_cmd(2, [[2]], temperature=0.3)
    results = _loop(w, [_rollout_cmd(1, [[1] * 3]), hot])
    assert [r.request_id for r in results] == [1, 2, -1]

    w = ScriptedWorker()
    w.engine.max_model_len = 8
    too_long = _rollout_cmd(2, [[2] * 6], max_new=4)          # 6 + 4 > 8
    results = _loop(w, [_rollout_cmd(1, [[1] * 3], max_new=4), too_long])
    assert [r.request_id for r in results] == [1, 2, -1]
    assert sum(1 for e in w.log if isinstance(e, tuple) and e[0] == "engine") == 2


def test_seeded_requests_draw_from_streams_numbered_by_prompt_position():
    w = ScriptedWorker()
    _loop(w, [_rollout_cmd(1, [[1], [2], [3]], indices=[10, 11, 12], seed=7)])
    assert [r.stream for r in w.engine._requests.values()] == [10, 11, 12]


def test_cancel_ends_the_batch_and_reports_cancelled_rows():
    w = ScriptedWorker()
    results = _loop(w, [_rollout_cmd(1, [[1] * 50]), lambda: (w.engine.steps >= 2, Command(Op.CANCEL, 99))])
    assert [r.request_id for r in results] == [99, 1, -1] and w.engine.cancelled
    assert results[1].payload.finish_reasons == ["cancelled"] and results[1].payload.tokens == [[]]
    assert w.engine.steps < 50


def test_shared_cancel_flags_stop_the_batch():
    import torch

    w = ScriptedWorker()
    cmd = _rollout_cmd(1, [[1] * 50])
    cmd.payload.cancel_flags = torch.tensor([True])
    results = _loop(w, [cmd])
    assert w.engine.cancelled and results[0].payload.finish_reasons == ["cancelled"]


def test_tensor_parallel_and_expert_parallel_rollouts_run_blocking():
    for w in (ScriptedWorker(tp=2), ScriptedWorker(ep=2)):
        results = _loop(w, [_rollout_cmd(1, [[1, 1]])])
        assert results[0].payload.tokens == [[9]] and ("rollout", 1, 4) in w.log
        assert not any(isinstance(e, tuple) and e[0] == "engine" for e in w.log)


def test_failures_travel_as_tracebacks_and_the_loop_survives():
    w = ScriptedWorker()
    w.train = lambda packs, acc: (_ for _ in ()).throw(RuntimeError("out of pages"))
    results = _loop(w, [Command(Op.TRAIN, 1, TrainPayload([[{}]], None)), Command(Op.MODEL_INFO, 2)])
    assert [(r.request_id, r.ok) for r in results] == [(1, False), (2, True), (-1, True)]
    assert "RuntimeError: out of pages" in results[0].error and results[0].payload is None


def test_queue_getter_modes():
    import queue

    q = queue.Queue()
    get = make_queue_getter(q)
    assert get(0.0) is None and get(0.01) is None
    q.put("a")
    q.put("b")
    assert get(0.0) == "a" and get(None) == "b"
