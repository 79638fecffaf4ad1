"""Agent loop of DuelGrid: every model turn sees the map, both status lines and the legal JSON actions and
must answer with one of them (plain text, no tools); the scripted opponent moves after each turn.

    areno train --algo gspo --ckpt <model> --dataset-path duelgrid:256 \
        --dataset-loader-fn examples/agentic/duelgrid/dataset_loader.py \
        --agent-fn examples/agentic/duelgrid/run_agent.py --reward-fn-path examples/agentic/duelgrid/reward.py
"""

from __future__ import annotations

import asyncio
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import game  # noqa: E402

from areno_b200.api.agentic import AgentTrajectory, AgentTrajectoryTurn  # noqa: E402


async def _episode(session, item) -> AgentTrajectory:
    state = item.record["state"]
    messages = [{"role": "system", "content": item.prompt}]
    turns = []
    while game.outcome(state) is None:
        legal = game.legal_actions(state, "A")
        messages.append({"role": "user", "content": f"{game.render(state)}\nLegal actions: {json.dumps(legal)}"})
        response = await session.complete_chat({"messages": messages, "model": "policy"})
        turns.append(AgentTrajectoryTurn(item=item, messages=list(messages), response=response))
        text = response["choices"][0]["message"].get("content") or ""
        messages.append({"role": "assistant", "content": text})
        state, _legal = game.step(state, text)
    return AgentTrajectory(turns=turns)


async def run_agent(session, batch):
    return await asyncio.gather(*[_episode(session, item) for item in batch.iter_samples()])
