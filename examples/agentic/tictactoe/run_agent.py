"""Agent loop for ``areno train --agent-fn``: plays one game per (prompt, sample) against the rule
opponent by calling the policy through the session's OpenAI-compatible endpoint with one tool.

    areno train --algo grpo --ckpt <model> --dataset-path tictactoe:256 \
        --dataset-loader-fn examples/agentic/tictactoe/dataset_loader.py \
        --agent-fn examples/agentic/tictactoe/run_agent.py --reward-fn-path examples/agentic/tictactoe/reward.py
"""

from __future__ import annotations

import asyncio
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from game import opponent_move, render, winner  # noqa: E402

from areno_b200.api.agentic import AgentTrajectory, AgentTrajectoryTurn  # noqa: E402

TOOLS = [{"type": "function", "function": {
    "name": "place_mark", "description": "Place your X on a free cell.",
    "parameters": {"type": "object", "properties": {"cell": {"type": "integer", "minimum": 0, "maximum": 8}},
                   "required": ["cell"]}}}]
MAX_TURNS = 5


async def _play(session, item) -> AgentTrajectory:
    board = ["."] * 9
    messages = [{"role": "system", "content": "You are X. Cells are numbered 0-8 row by row."},
                {"role": "user", "content": f"{item.prompt}\n\nBoard:\n{render(board)}"}]
    turns = []
    outcome = "unfinished"
    for _ in range(MAX_TURNS):
        response = await session.complete_chat({"messages": messages, "tools": TOOLS, "model": "policy"})
        turns.append(AgentTrajectoryTurn(item=item, messages=list(messages), response=response, tools=TOOLS))
        choice = response["choices"][0]["message"]
        calls = choice.get("tool_calls") or []
        if not calls:
            outcome = "no_move"
            break
        messages.append({"role": "assistant", "content": None, "tool_calls": calls})
        try:
            cell = int(json.loads(calls[0]["function"]["arguments"])["cell"])
        except (KeyError, ValueError, TypeError):
            cell = -1
        if not 0 <= cell < 9 or board[cell] != ".":
            messages.append({"role": "tool", "tool_call_id": calls[0].get("id"), "name": "place_mark",
                             "content": json.dumps({"error": "illegal move", "result": "loss"})})
            outcome = "illegal"
            break
        board[cell] = "X"
        state = winner(board)
        if state is None:
            board[opponent_move(board)] = "O"
            state = winner(board)
        result = {"X": "win", "O": "loss", "draw": "draw"}.get(state or "", "continue")
        messages.append({"role": "tool", "tool_call_id": calls[0].get("id"), "name": "place_mark",
                         "content": json.dumps({"board": render(board), "result": result})})
        if state is not None:
            outcome = result
            break
    item.record["outcome"] = outcome
    return AgentTrajectory(turns=turns)


async def run_agent(session, batch):
    return await asyncio.gather(*[_play(session, item) for item in batch.iter_samples()])
