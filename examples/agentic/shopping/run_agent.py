"""Agent loop of the shopping task: up to six model turns with four tools; the environment answers each
tool call from the rule engine and records the submitted bundle for the reward.

    areno train --algo gspo --ckpt <model> --dataset-path shopping:2048 \
        --dataset-loader-fn examples/agentic/shopping/dataset_loader.py \
        --agent-fn examples/agentic/shopping/run_agent.py --reward-fn-path examples/agentic/shopping/reward.py
"""

from __future__ import annotations

import asyncio
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import game  # noqa: E402

from areno_b200.api.agentic import AgentTrajectory, AgentTrajectoryTurn  # noqa: E402


def _tool(name, desc, props, required):
    return {"type": "function", "function": {"name": name, "description": desc,
                                             "parameters": {"type": "object", "properties": props, "required": required}}}


_IDS = {"type": "array", "items": {"type": "string"}}
TOOLS = [
    _tool("search_catalog", "List item ids and prices of one category.", {"category": {"type": "string"}}, ["category"]),
    _tool("inspect_items", "Show category, price and features of items.", {"ids": _IDS}, ["ids"]),
    _tool("check_kit", "Check a candidate bundle against the task.", {"ids": _IDS}, ["ids"]),
    _tool("submit_bundle", "Submit the final bundle.", {"ids": _IDS}, ["ids"]),
]
MAX_TURNS = 6


def _answer(task, name, args, used):
    used.append(name)
    if name == "search_catalog":
        return {"items": game.search(task, str(args.get("category", "")))}
    ids = [str(i) for i in (args.get("ids") or [])]
    if name == "inspect_items":
        return {"items": game.inspect(task, ids)}
    if name == "check_kit":
        return game.check(task, ids)
    if name == "submit_bundle":
        return dict(game.check(task, ids), submitted=ids, tools_used=list(used))
    return {"error": f"unknown tool {name}"}


async def _episode(session, item) -> AgentTrajectory:
    task = item.record["task"]
    messages = [{"role": "system", "content": "You are a careful shopping assistant. Always answer with a tool call."},
                {"role": "user", "content": item.prompt}]
    turns, used = [], []
    for _ in range(MAX_TURNS):
        response = await session.complete_chat({"messages": messages, "tools": TOOLS, "model": "policy"})
        turns.append(AgentTrajectoryTurn(item=item, messages=list(messages), response=response, tools=TOOLS))
        calls = response["choices"][0]["message"].get("tool_calls") or []
        if not calls:
            break
        messages.append({"role": "assistant", "content": None, "tool_calls": calls})
        done = False
        for call in calls:
            name = call["function"]["name"]
            try:
                args = json.loads(call["function"].get("arguments") or "{}")
            except ValueError:
                args = {}
            result = _answer(task, name, args if isinstance(args, dict) else {}, used)
            messages.append({"role": "tool", "tool_call_id": call.get("id"), "name": name, "content": json.dumps(result)})
            done = done or name == "submit_bundle"
        if done:
            break
    return AgentTrajectory(turns=turns)


async def run_agent(session, batch):
    return await asyncio.gather(*[_episode(session, item) for item in batch.iter_samples()])
