"""Wire protocol between the engine coordinator (driver) and the rank workers.

Commands carry an ``Op``, a request id (for demultiplexing concurrent async calls) and a payload
dataclass; results carry either a payload or a formatted traceback.  The same objects are used by
every cluster flavour: spawned processes (pickled through ``multiprocessing`` queues), the
in-process worker thread, and SPMD ranks under ``torch.distributed.run``.
Role of ``areno/engine/protocol.py:31-151`` in the reference.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field, replace
from typing import Any

from .inference import SamplingParams


class Op(enum.Enum):
    INFER_ROLLOUT = "infer_rollout"
    TRAIN = "train"
    SCORE_LOGPROBS = "score_logprobs"
    SCORE_VALUES = "score_values"
    SCORE_REWARDS = "score_rewards"
    TRAIN_VALUES = "train_values"
    ENSURE_ROLES = "ensure_roles"
    SAVE_CHECKPOINT = "save_checkpoint"
    ROLLOUT_SESSION_BEGIN = "rollout_session_begin"
    ROLLOUT_SESSION_SYNC = "rollout_session_sync"
    ROLLOUT_SESSION_END = "rollout_session_end"
    PROBE_ROLLOUT_CACHE = "probe_rollout_cache"
    PROBE_TRAIN_MEMORY = "probe_train_memory"
    MODEL_INFO = "model_info"
    CANCEL = "cancel"
    SHUTDOWN = "shutdown"


@dataclass
class Command:
    op: Op
    request_id: int = 0
    payload: Any = None
    result_ranks: tuple[int, ...] | None = None  # ranks whose result the caller waits for (None = all)


@dataclass
class WorkerResult:
    rank: int
    request_id: int = 0
    ok: bool = True
    payload: Any = None
    error: str | None = None
    partial: bool = False  # an early per-request result from a continuous rollout


@dataclass
class RolloutPayload:
    prompts_by_dp: list[list[list[int]]]
    prompt_indices_by_dp: list[list[int]]
    max_new_tokens: int
    eos_token_ids: tuple[int, ...] = ()
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    max_running_seqs: int = 64
    max_cache_len: int = 0
    decode_progress_interval_s: float = 0.0
    cancel_flags: Any = None            # shared-memory bool tensor, one flag per global prompt index
    session_key: tuple | None = None    # payloads with equal keys may share one running batch

    def compatibility_key(self) -> tuple:
        p = self.sampling_params
        return (self.max_new_tokens, tuple(self.eos_token_ids), p.temperature, p.top_p, p.top_k, p.min_new_tokens,
                tuple(p.stop_token_ids), tuple(p.suppress_token_ids), self.cancel_flags is None)


@dataclass
class TrainPayload:
    packs: list                 # list of micro-batches, each a list of per-DP-rank shards
    gradient_accumulation_steps: int | None = None


@dataclass
class ScorePayload:
    role: str
    rows_by_dp: list[list[list[int]]]
    pad_token_id: int = 0
    microbatch_size: int = 8


@dataclass
class TrainValuesPayload:
    role: str
    packs: list
    gradient_accumulation_steps: int | None = None
    cliprange_value: float = 0.5
    value_loss_coef: float = 0.5


@dataclass
class RolesPayload:
    roles: dict


@dataclass
class CachePayload:
    max_running_seqs: int
    max_cache_len: int


@dataclass
class SavePayload:
    path: str


def narrow_for_rank(payload: Any, *, train_dp_rank: int, rollout_dp_rank: int) -> Any:
    """The part of a payload that one rank reads.  Payloads carry one entry per data-parallel row (prompts, score
    rows, training shards) and a worker only ever looks at its own row's, so a driver that ships commands to worker
    processes blanks the others instead of serialising the whole job's data once per rank.  The shape stays the
    same (a list with one slot per row), so workers index it as before."""
    def only(rows, keep, empty):
        return [row if i == keep else empty() for i, row in enumerate(rows)]

    if isinstance(payload, RolloutPayload):
        return replace(payload, prompts_by_dp=only(payload.prompts_by_dp, rollout_dp_rank, list),
                       prompt_indices_by_dp=only(payload.prompt_indices_by_dp, rollout_dp_rank, list))
    if isinstance(payload, ScorePayload):
        return replace(payload, rows_by_dp=only(payload.rows_by_dp, train_dp_rank, list))
    if isinstance(payload, (TrainPayload, TrainValuesPayload)):
        packs = [only(shards, train_dp_rank, lambda: None) if isinstance(shards, (list, tuple)) else shards
                 for shards in payload.packs]
        return replace(payload, packs=packs)
    return payload
