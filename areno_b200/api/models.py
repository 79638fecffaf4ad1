"""Wire-format models of the SDK: what rollouts return and what training consumes.

Field-for-field compatible with ``areno/api/models.py`` of the reference (pydantic models), so
algorithm scripts written against it run unchanged.
"""

from __future__ import annotations

from enum import Enum

from pydantic import BaseModel, Field


class BackendType(Enum):
    Areno = "Areno"


class SamplingParams(BaseModel):
    """Generation controls.  ``greedy`` forces temperature 0; ``top_k=-1`` disables top-k;
    ``max_context_len`` caps whole agentic trajectories (prompt plus every generated turn)."""

    greedy: bool = False
    top_p: float = 1.0
    top_k: int = -1
    max_new_tokens: int = 16
    max_context_len: int | None = None
    temperature: float = 1.0
    stop: list[str] | None = None
    stop_token_ids: list[int] | None = None
    ignore_eos: bool = False
    skip_special_tokens: bool = True
    max_prompt_len: int | None = None
    # additions to the reference's fields: EOS / stop ids are masked out for the first ``min_new_tokens`` tokens;
    # with a ``seed`` every sample draws from a random stream numbered by its position in the request, so a rollout
    # is reproducible whatever else shares the running batch
    min_new_tokens: int = 0
    seed: int | None = None


class RolloutSequence(BaseModel):
    """One sampled completion; ``resp_logprobs[i]`` is the rollout-policy log-prob of ``resp_tokens[i]``."""

    resp_tokens: list[int] = Field(default_factory=list)
    resp_logprobs: list[float] = Field(default_factory=list)


class RolloutResult(BaseModel):
    sequences: list[RolloutSequence] = Field(default_factory=list)


class TrainSequence(BaseModel):
    """A rollout converted into a training sample: prompt + response tokens with per-token signals."""

    prompt_mask: list[bool] = Field(default_factory=list)
    loss_mask: list[bool] = Field(default_factory=list)
    tokens: list[int] = Field(default_factory=list)
    logprobs: list[float] = Field(default_factory=list)
    advantages: list[float] = Field(default_factory=list)
    returns: list[float] = Field(default_factory=list)
    values: list[float] = Field(default_factory=list)
    ref_logprobs: list[float] = Field(default_factory=list)
    reward: float = 0.0
    eos_token_id: int = 0
