"""Coding-agent loop: the task's files are written to a private temporary workspace, the policy works on it
through the tools of ``coding_tools.Workspace`` for a bounded number of turns, and ``submit`` runs the task's
test command one last time; its result is what the reward reads.

    areno train --algo gspo --ckpt <model> --dataset-path coding:100 \
        --dataset-loader-fn examples/agentic/coding/dataset_loader.py \
        --agent-fn examples/agentic/coding/run_agent.py --reward-fn-path examples/agentic/coding/reward.py
"""

from __future__ import annotations

import asyncio
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from agent_loop import MAX_TURNS, TOOLS, dispatch, run_episode  # noqa: E402,F401

from areno_b200.api.agentic import AgentTrajectory, AgentTrajectoryTurn  # noqa: E402

_dispatch = dispatch   # older name


async def _episode(session, item) -> AgentTrajectory:
    _messages, turns = await run_episode(session.complete_chat, item.record["task"], item.prompt)
    return AgentTrajectory(turns=[AgentTrajectoryTurn(item=item, messages=before, response=response, tools=TOOLS)
                                  for before, response in turns])


async def run_agent(session, batch):
    return await asyncio.gather(*[_episode(session, item) for item in batch.iter_samples()])
