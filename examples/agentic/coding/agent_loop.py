"""Tool loop of the coding agent, shared by the training entry point (``run_agent.py``) and the local command
line (``code_cli.py``): tool schemas, dispatch onto a ``coding_tools.Workspace`` and one bounded episode.

``run_episode`` only needs an async ``complete(payload) -> response`` callable speaking the chat-completions
format, so the same loop runs against the trainer's in-process session or an HTTP endpoint.
"""

from __future__ import annotations

import asyncio
import json
import os
import re
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from coding_tools import Workspace  # noqa: E402


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
SYSTEM_PROMPT = "You are a coding agent. Work only through tool calls."


def dispatch(ws: Workspace, task: dict, name: str, args: dict) -> dict:
    """Run one tool call.  ``submit`` runs the task's test command one last time; its result is what the reward reads."""
    try:
        if name == "submit":
            final = ws.run_command(task["test_command"])
            return {"status": args.get("status", "solved"), "tests_passed": final.get("returncode") == 0,
                    "output": final.get("output", final.get("error", ""))[-800:], "submitted": True}
        fn = getattr(ws, name, None)
        if fn is None or name.startswith("_") or name == "close":
            return {"error": f"unknown tool {name}"}
        return fn(**args)
    except (TypeError, ValueError, OSError, re.error) as exc:   # bad arguments are the policy's problem, not a crash
        return {"error": f"{type(exc).__name__}: {exc}"}


async def run_episode(complete, task: dict, prompt: str, max_turns: int = MAX_TURNS, on_turn=None, on_tool=None):
    """Play one task.  Returns ``(messages, turns)`` where ``turns`` is a list of ``(messages_before, response)``.

    ``on_turn(response)`` / ``on_tool(name, args, result)`` are optional observers (the command line prints with them)."""
    ws = Workspace(task["files"])
    messages = [{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": prompt}]
    turns = []
    try:
        for _ in range(max_turns):
            response = await complete({"messages": messages, "tools": TOOLS, "model": "policy"})
            turns.append((list(messages), response))
            if on_turn is not None:
                on_turn(response)
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
                args = args if isinstance(args, dict) else {}
                result = await asyncio.to_thread(dispatch, ws, task, name, args)
                if on_tool is not None:
                    on_tool(name, args, result)
                messages.append({"role": "tool", "tool_call_id": call.get("id"), "name": name, "content": json.dumps(result)})
                done = done or name == "submit"
            if done:
                break
    finally:
        ws.close()
    return messages, turns
