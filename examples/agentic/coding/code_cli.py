"""Run the coding agent outside training: one task against a served model, transcript on the terminal.

    python examples/agentic/coding/code_cli.py --base-url http://127.0.0.1:8000/v1 --task 3
    python examples/agentic/coding/code_cli.py --base-url http://127.0.0.1:8000/v1 --dataset examples/agentic/coding/dataset.jsonl --task 0
    python examples/agentic/coding/code_cli.py --dump-dataset /tmp/coding.jsonl --n 200       # write generated tasks
    python examples/agentic/coding/code_cli.py --reference-fix --task 3                       # no model: apply the known fix

The endpoint is any OpenAI-compatible ``/chat/completions`` server with tool calling (``areno serve``).  The exit
code is 0 when the task's tests pass after ``submit``.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import sys
import urllib.request

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from agent_loop import run_episode  # noqa: E402
from tasks import make_task  # noqa: E402

PROMPT = ("Fix the bug described below in the repository. Inspect files, edit them, run the tests and then call "
          "submit.\n\nIssue: {issue}")


def http_complete(base_url: str, model: str, api_key: str = "none", timeout_s: float = 600.0):
    """An async ``complete(payload)`` that posts to ``<base_url>/chat/completions``."""

    def post(payload: dict) -> dict:
        body = dict(payload, model=model)
        req = urllib.request.Request(base_url.rstrip("/") + "/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json", "Authorization": f"Bearer {api_key}"})
        with urllib.request.urlopen(req, timeout=timeout_s) as resp:
            return json.loads(resp.read())

    async def complete(payload: dict) -> dict:
        return await asyncio.to_thread(post, payload)

    return complete


def scripted_fix(task: dict):
    """A stand-in policy that applies the task's reference fix and submits (checks the plumbing without a model)."""
    script = [("write_file", {"path": path, "content": content}) for path, content in task["reference_fix"].items()]
    script += [("run_command", {"command": task["test_command"]}), ("submit", {"status": "solved"})]
    state = {"i": 0}

    async def complete(payload: dict) -> dict:
        name, args = script[min(state["i"], len(script) - 1)]
        state["i"] += 1
        return {"choices": [{"message": {"role": "assistant", "content": None, "tool_calls": [
            {"id": f"call{state['i']}", "type": "function", "function": {"name": name, "arguments": json.dumps(args)}}]}}]}

    return complete


def load_task(dataset: str | None, index: int) -> dict:
    if dataset:
        with open(dataset) as f:
            rows = [json.loads(line) for line in f if line.strip()]
        return rows[index % len(rows)]
    return make_task(index)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--base-url", default=None)
    ap.add_argument("--model", default="policy")
    ap.add_argument("--dataset", default=None, help="JSONL of task records (default: generated tasks)")
    ap.add_argument("--task", type=int, default=0)
    ap.add_argument("--max-turns", type=int, default=10)
    ap.add_argument("--reference-fix", action="store_true", help="apply the task's known fix instead of asking a model")
    ap.add_argument("--dump-dataset", default=None, help="write --n generated tasks to this JSONL file and exit")
    ap.add_argument("--n", type=int, default=100)
    args = ap.parse_args(argv)
    if args.dump_dataset:
        with open(args.dump_dataset, "w") as f:
            for i in range(args.n):
                f.write(json.dumps(make_task(i)) + "\n")
        print(f"wrote {args.n} tasks to {args.dump_dataset}")
        return 0
    task = load_task(args.dataset, args.task)
    if args.reference_fix:
        complete = scripted_fix(task)
    elif args.base_url:
        complete = http_complete(args.base_url, args.model)
    else:
        ap.error("give --base-url, or --reference-fix to run without a model")
    print(f"task {task['instance_id']}: {task['problem_statement']}\n")
    outcome = {"passed": False}

    def on_turn(response):
        text = response["choices"][0]["message"].get("content")
        if text:
            print(f"assistant: {text}")

    def on_tool(name, targs, result):
        shown = json.dumps(result)
        print(f"  {name}({json.dumps(targs)[:160]}) -> {shown[:300]}{'...' if len(shown) > 300 else ''}")
        if name == "submit":
            outcome["passed"] = bool(result.get("tests_passed"))

    asyncio.run(run_episode(complete, task, PROMPT.format(issue=task["problem_statement"]), args.max_turns, on_turn, on_tool))
    print("\nresult:", "tests pass" if outcome["passed"] else "tests do not pass")
    return 0 if outcome["passed"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
