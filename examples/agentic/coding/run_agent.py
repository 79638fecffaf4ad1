"""Coding-agent loop: the task's files are written to a private temporary workspace, the policy works on it
through the tools of ``coding_tools.Workspace`` for a bounded number of turns, and ``submit`` runs the task's
test command one last time; its result is what the reward reads.

    areno train --algo gspo --ckpt <model> --dataset-path coding:100 \
        --dataset-loader-fn examples/agentic/coding/dataset_loader.py \
        --agent-fn examples/agentic/coding/run_agent.py --reward-fn-path examples/agentic/coding/reward.py
"""

from __future__ import annotations

import asyncio
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from coding_tools import Workspace  # noqa: E402

from areno_b200.api.agentic import AgentTrajectory, AgentTrajectoryTurn  # noqa: E402


def _tool(name, desc, props, required=()):
    return {"type": "function", "function": {"name": name, "description": desc, "parameters": {
        "type": "object", "properties": props, "required": list(required)}}}


_S = {"type": "string"}
TOOLS = [
    _tool("list_files", "List the files of the repository.", {}),
    _tool("read_file", "Read a line range of a file.", {"path": _S, "start": {"type": "integer"}, "end": {"type": "integer"}}, ["path"]),
    _tool("rg", "Regex search over the repository.", {"pattern": _S}, ["pattern"]),
    _tool("replace_text", "Replace one exact occurrence of text in a file.", {"path": _S, "old": _S, "new": _S}, ["path", "old", "new"]),
    _tool("write_file", "Create or overwrite a file.", {"path": _S, "content": _S}, ["path", "content"]),
    _tool("run_command", "Run a short shell command (tests) in the repository.", {"command": _S}, ["command"]),
    _tool("submit", "Finish: report 'solved' or 'blocked'.", {"status": _S, "summary": _S}, ["status"]),
]
MAX_TURNS = 10


def _dispatch(ws: Workspace, task: dict, name: str, args: dict) -> dict:
    try:
        if name == "submit":
            final = ws.run_command(task["test_command"])
            return {"status": args.get("status", "solved"), "tests_passed": final.get("returncode") == 0,
                    "output": final.get("output", final.get("error", ""))[-800:], "submitted": True}
        fn = getattr(ws, name, None)
        if fn is None or name.startswith("_") or name == "close":
            return {"error": f"unknown tool {name}"}
        return fn(**args)
    except (TypeError, ValueError, OSError, re_error) as exc:   # bad arguments are the policy's problem, not a crash
        return {"error": f"{type(exc).__name__}: {exc}"}


import re  # noqa: E402

re_error = re.error


async def _episode(session, item) -> AgentTrajectory:
    task = item.record["task"]
    ws = Workspace(task["files"])
    messages = [{"role": "system", "content": "You are a coding agent. Work only through tool calls."},
                {"role": "user", "content": item.prompt}]
    turns = []
    try:
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
                result = await asyncio.to_thread(_dispatch, ws, task, name, args if isinstance(args, dict) else {})
                messages.append({"role": "tool", "tool_call_id": call.get("id"), "name": name, "content": json.dumps(result)})
                done = done or name == "submit"
            if done:
                break
    finally:
        ws.close()
    return AgentTrajectory(turns=turns)


async def run_agent(session, batch):
    return await asyncio.gather(*[_episode(session, item) for item in batch.iter_samples()])
