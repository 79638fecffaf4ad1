"""Command execution inside a rank worker: op dispatch and the continuous-rollout loop.

``execute(worker, cmd)`` runs one command to completion.  ``WorkerLoop`` wraps it for the queue-fed
flavours (worker thread or spawned process): while a rollout is decoding it keeps draining the
command queue, and further ``INFER_ROLLOUT`` commands whose sampling setup is compatible join the
running batch between decode steps (continuous batching across requests); each request's result
is sent back as soon as its own rows have finished.  Anything else waits until the batch drains.

Role of ``ArenoWorker.handle`` / ``run_continuous_rollout_payload`` in the reference
(``areno/engine/worker.py:97-275``).
"""

from __future__ import annotations

import queue
import traceback
from typing import Any, Callable

from ..parallel.context import get_context
from .inference import RolloutOutput
from .protocol import Command, Op, RolloutPayload, WorkerResult


def execute(worker, cmd: Command) -> Any:
    """Run a non-rollout command (or a rollout to completion) and return its payload."""
    op, p = cmd.op, cmd.payload
    ctx = get_context()
    if op == Op.INFER_ROLLOUT:
        return _rollout_blocking(worker, p)
    if op == Op.TRAIN:
        return worker.train(p.packs, p.gradient_accumulation_steps)
    if op == Op.ROLLOUT_SESSION_BEGIN:
        worker.prepare_actor_onloaded()
        return None
    if op == Op.ROLLOUT_SESSION_SYNC:
        return None
    if op == Op.ROLLOUT_SESSION_END:
        worker.prepare_for_train()
        return None
    if op == Op.ENSURE_ROLES:
        return worker.role_manager().ensure_roles(p.roles)
    if op == Op.SCORE_LOGPROBS:
        return worker.role_manager().score_logprobs(p.role, p.rows_by_dp[ctx.dp_rank], p.pad_token_id, p.microbatch_size)
    if op == Op.SCORE_VALUES:
        return worker.role_manager().score_values(p.role, p.rows_by_dp[ctx.dp_rank], p.pad_token_id)
    if op == Op.SCORE_REWARDS:
        return worker.role_manager().score_rewards(p.role, p.rows_by_dp[ctx.dp_rank], p.pad_token_id)
    if op == Op.TRAIN_VALUES:
        return worker.role_manager().train_values(p.role, p.packs, p.gradient_accumulation_steps,
                                                  cliprange_value=p.cliprange_value, value_loss_coef=p.value_loss_coef)
    if op == Op.SAVE_CHECKPOINT:
        worker.save_checkpoint(p.path)
        return p.path
    if op == Op.PROBE_ROLLOUT_CACHE:
        return worker.probe_rollout_cache(p.max_running_seqs, p.max_cache_len)
    if op == Op.PROBE_TRAIN_MEMORY:
        return worker.peak_memory_fraction()
    if op == Op.MODEL_INFO:
        return worker.model_info()
    if op == Op.CANCEL:
        if worker.infer is not None and worker.infer.sched is not None:
            worker.infer.cancel_all()
        return None
    raise ValueError(f"unsupported op {op}")


def _local_rows(p: RolloutPayload, worker=None):
    """Rollout prompts are split over the data-parallel rows of the ROLLOUT layout."""
    ctx = worker.rollout_ctx if worker is not None else get_context().rollout_layout
    return p.prompts_by_dp[ctx.dp_rank], p.prompt_indices_by_dp[ctx.dp_rank]


def _rollout_blocking(worker, p: RolloutPayload) -> RolloutOutput:
    prompts, indices = _local_rows(p, worker)
    if not prompts and worker.rollout_ctx.ep_size == 1:
        return RolloutOutput(prompt_indices=[])
    # expert parallel: a rank without prompts still joins every forward pass of the others (idle passes)
    out = worker.rollout(prompts, p.sampling_params, p.eos_token_ids, p.max_new_tokens, max_running=p.max_running_seqs,
                         progress_interval_s=p.decode_progress_interval_s, stream_ids=list(indices))
    out.prompt_indices = list(indices)
    return out


class WorkerLoop:
    """Queue-fed command loop with continuous batching across rollout requests."""

    def __init__(self, worker, rank: int, get_cmd: Callable[[float | None], Command | None],
                 put_result: Callable[[WorkerResult], None]):
        self.worker = worker
        self.rank = rank
        self.get_cmd = get_cmd          # get_cmd(timeout) -> Command | None (None on timeout)
        self.put_result = put_result
        self.deferred: list[Command] = []

    def run(self) -> None:
        while True:
            cmd = self.deferred.pop(0) if self.deferred else self.get_cmd(None)
            if cmd is None:
                continue
            if cmd.op == Op.SHUTDOWN:
                self.put_result(WorkerResult(self.rank, cmd.request_id, True, None))
                return
            try:
                rctx = self.worker.rollout_ctx
                # request-concurrent batching needs engines that may step on their own: not with tensor-parallel
                # rollout nor with expert parallelism, whose ranks exchange tokens in every forward pass
                if cmd.op == Op.INFER_ROLLOUT and rctx.tp_size == 1 and rctx.ep_size == 1:
                    self._continuous_rollout(cmd)
                else:
                    self.put_result(WorkerResult(self.rank, cmd.request_id, True, execute(self.worker, cmd)))
            except BaseException:  # noqa: BLE001 - the traceback travels to the driver
                self.put_result(WorkerResult(self.rank, cmd.request_id, False, None, traceback.format_exc()))

    # ------------------------------------------------------------- rollout loop
    def _continuous_rollout(self, first: Command) -> None:
        worker = self.worker
        p0: RolloutPayload = first.payload
        key = p0.compatibility_key()
        worker.prepare_for_rollout()
        rows0, _ = _local_rows(p0, worker)
        longest = max((len(r) for r in rows0), default=1) + p0.max_new_tokens
        eng = worker.inference_engine(max(p0.max_running_seqs, 1), max((longest + 63) // 64 * 64,
                                                                        p0.max_cache_len or 0))
        eng.begin(p0.sampling_params, p0.eos_token_ids, p0.max_new_tokens)
        pending: dict[int, dict] = {}

        def admit(cmd: Command) -> None:
            rows, indices = _local_rows(cmd.payload, self.worker)
            state = {"cmd": cmd, "indices": list(indices), "left": len(rows), "reqs": []}
            if not rows:                     # nothing for this data-parallel row: acknowledge once, track nothing
                self._finish(state)
                return
            pending[cmd.request_id] = state
            seeded = cmd.payload.sampling_params.seed is not None
            for r, idx in zip(rows, indices):
                # a seeded request reproduces: its rows draw from streams numbered by their position
                rid = eng.add_request(r, cmd.payload.max_new_tokens, tag=cmd.request_id,
                                      stream=int(idx) if seeded else None)
                state["reqs"].append(rid)

        admit(first)
        blocked = False
        while pending:
            if not blocked:
                # drain newly arrived commands without blocking the decode loop
                while True:
                    nxt = self.get_cmd(0.0)
                    if nxt is None:
                        break
                    if nxt.op == Op.INFER_ROLLOUT and nxt.payload.compatibility_key() == key \
                            and self._fits(eng, nxt.payload):
                        admit(nxt)
                    elif nxt.op == Op.CANCEL:
                        eng.cancel_all()
                        self.put_result(WorkerResult(self.rank, nxt.request_id, True, None))
                    else:
                        self.deferred.append(nxt)
                        blocked = True  # preserve command order: stop admitting behind it
                        break
            cancel = p0.cancel_flags
            if cancel is not None and bool(cancel.any()):
                eng.cancel_all()
            for req in eng.step():
                state = pending.get(req.tag)
                if state is None:
                    continue
                state["left"] -= 1
                if state["left"] == 0:
                    self._finish(state, eng)
                    del pending[req.tag]
            if eng.idle and pending:
                for state in list(pending.values()):
                    self._finish(state, eng)
                pending.clear()

    @staticmethod
    def _fits(eng, payload: RolloutPayload) -> bool:
        rows = payload.prompts_by_dp[get_context().rollout_layout.dp_rank]
        longest = max((len(r) for r in rows), default=1) + payload.max_new_tokens
        return longest <= eng.max_model_len

    def _finish(self, state: dict, eng=None) -> None:
        cmd = state["cmd"]
        out = RolloutOutput(prompt_indices=state["indices"])
        for rid in state["reqs"]:
            req = eng._requests[rid]
            out.tokens.append(req.tokens or [])
            out.logprobs.append(req.logprobs or [])
            out.finish_reasons.append(req.reason or "cancelled")
        self.put_result(WorkerResult(self.rank, cmd.request_id, True, out))


def make_queue_getter(q) -> Callable[[float | None], Command | None]:
    def get(timeout: float | None):
        try:
            if timeout is None:
                return q.get()
            if timeout <= 0:
                return q.get_nowait()
            return q.get(timeout=timeout)
        except queue.Empty:
            return None

    return get
