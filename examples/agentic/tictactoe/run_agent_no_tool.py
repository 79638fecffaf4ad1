"""One-step agent: one chat completion per position, the answer is a ``<move>N</move>`` tag (no tools).

    python examples/agentic/tictactoe/dataset_generator.py --out /tmp/ttt.jsonl --n 2000
    areno train --algo grpo --ckpt <model> --dataset-path /tmp/ttt.jsonl \
        --dataset-loader-fn examples/agentic/tictactoe/dataset_loader_no_tool.py \
        --agent-fn examples/agentic/tictactoe/run_agent_no_tool.py \
        --reward-fn-path examples/agentic/tictactoe/reward_no_tool.py
"""

from __future__ import annotations

import asyncio

from areno_b200.api.agentic import AgentTrajectory, AgentTrajectoryTurn

SYSTEM_PROMPT = ("You are a careful tic-tac-toe player and you play X. Numbers on the board are free squares, not "
                 "marks. Take a win if there is one; otherwise stop O from completing a row; otherwise pick any free "
                 "square. Reply with exactly one tag such as <move>5</move>.")


async def _one(session, item) -> AgentTrajectoryTurn:
    messages = [{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": item.prompt}]
    response = await session.complete_chat({"messages": messages, "model": "policy"})
    return AgentTrajectoryTurn(item=item, messages=messages, response=response)


async def run_agent(session, batch):
    """All positions of the batch in flight at once; the engine batches them."""
    turns = await asyncio.gather(*[_one(session, item) for item in batch.iter_samples()])
    return [AgentTrajectory(turns=[t]) for t in turns]
