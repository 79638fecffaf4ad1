"""The shopping, DuelGrid and coding examples driven end to end by a scripted stand-in for the policy:
agent loop, rule engines, tool plumbing and rewards (no model, no GPU)."""

from __future__ import annotations

import asyncio
import importlib.util
import json
import sys
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parents[1]


def _load(path: Path, name: str):
    for mod in ("game", "tasks", "coding_tools", "dataset_generator", "reward_no_tool"):      # each example ships its own helper modules of these names
        sys.modules.pop(mod, None)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class ScriptedSession:
    """``complete_chat`` answers from a policy function of the conversation so far."""

    def __init__(self, policy):
        self.policy, self.calls = policy, 0

    async def complete_chat(self, payload):
        self.calls += 1
        message = self.policy(payload["messages"])
        return {"choices": [{"message": message}], "areno": {"response_tokens": [5, 6], "response_logprobs": [-0.1, -0.2]}}


def _batch(rows):
    from areno_b200.api.agentic import AgentItem

    items = [AgentItem(record=r, prompt=r["prompt"], input_tokens=[1, 2, 3], prompt_index=i, sample_index=0)
             for i, r in enumerate(rows)]
    return SimpleNamespace(iter_samples=lambda: iter(items))


def _call(name, args, cid="c1"):
    return {"role": "assistant", "content": None,
            "tool_calls": [{"id": cid, "type": "function", "function": {"name": name, "arguments": json.dumps(args)}}]}


def _record(traj, source):
    """What the trainer hands to a reward function, rebuilt from the last turn of a trajectory."""
    from areno_b200.api.agentic import tool_results_from_messages

    last = traj.turns[-1]
    messages = list(last.messages) + [last.response["choices"][0]["message"]]
    return SimpleNamespace(messages=messages, tool_results=tool_results_from_messages(messages), source_record=source)


def test_shopping_example():
    ex = ROOT / "examples/agentic/shopping"
    rows = _load(ex / "dataset_loader.py", "shop_loader").load_training_dataset(
        "shopping:3", default_loader=None, load_dataset=None, load_from_disk=None)
    assert len(rows) == 3 and rows[0]["task"]["categories"]
    agent = _load(ex / "run_agent.py", "shop_agent")
    game = sys.modules["game"]
    task = rows[0]["task"]

    def solve(task):
        for combo in __import__("itertools").product(*[[it["id"] for it in task["catalog"] if it["category"] == c]
                                                        for c in task["categories"]]):
            if game.check(task, list(combo))["ok"]:
                return list(combo)
        raise AssertionError("generated task has no solution")

    bundle = solve(task)

    def policy(messages):
        step = sum(1 for m in messages if m["role"] == "assistant")
        plan = [("search_catalog", {"category": task["categories"][0]}), ("inspect_items", {"ids": bundle}),
                ("check_kit", {"ids": bundle}), ("submit_bundle", {"ids": bundle})]
        return _call(*plan[step])

    trajs = asyncio.run(agent.run_agent(ScriptedSession(policy), _batch(rows[:1])))
    assert len(trajs) == 1 and len(trajs[0].turns) == 4
    final_messages = trajs[0].turns[-1].messages
    assert [m["name"] for m in final_messages if m["role"] == "tool"] == ["search_catalog", "inspect_items", "check_kit"]
    reward = _load(ex / "reward.py", "shop_reward").reward_fn
    # the record the trainer builds ends with the last assistant call; append the tool answer the loop produced
    done = [{"name": "submit_bundle", "content": json.dumps(dict(game.check(task, bundle), submitted=bundle,
             tools_used=["search_catalog", "inspect_items", "check_kit", "submit_bundle"]))}]
    assert reward(SimpleNamespace(tool_results=done)) == 1.0
    assert reward(SimpleNamespace(tool_results=[{"content": json.dumps(dict(game.check(task, bundle), submitted=bundle,
                                                                        tools_used=["submit_bundle"]))}])) == 0.6
    assert reward(SimpleNamespace(tool_results=[])) == 0.0


def test_duelgrid_example():
    ex = ROOT / "examples/agentic/duelgrid"
    rows = _load(ex / "dataset_loader.py", "duel_loader").load_training_dataset(
        "duelgrid:2", default_loader=None, load_dataset=None, load_from_disk=None)
    agent = _load(ex / "run_agent.py", "duel_agent")
    game = sys.modules["game"]

    def policy(messages):      # attack when offered, otherwise the first legal move, sometimes garbage
        legal = json.loads(messages[-1]["content"].split("Legal actions: ")[1])
        if len([m for m in messages if m["role"] == "assistant"]) == 1:
            return {"role": "assistant", "content": "I will teleport"}
        pick = {"action": "attack"} if {"action": "attack"} in legal else legal[-1]
        return {"role": "assistant", "content": f"My move: {json.dumps(pick)}"}

    session = ScriptedSession(policy)
    trajs = asyncio.run(agent.run_agent(session, _batch(rows)))
    assert len(trajs) == 2 and all(1 <= len(t.turns) <= 16 for t in trajs)
    reward = _load(ex / "reward.py", "duel_reward").reward_fn
    for traj, row in zip(trajs, rows):
        rec = _record(traj, row)
        value = reward(rec)
        answers = [m["content"] for m in rec.messages if m["role"] == "assistant"]
        final = game.replay(row["state"], answers)
        assert final["outcome"] in ("win", "loss", "draw") and final["illegal"] == 1 and 0.0 <= value <= 1.3
    assert reward(SimpleNamespace(messages=[], source_record={})) == 0.0


def test_coding_example():
    ex = ROOT / "examples/agentic/coding"
    rows = _load(ex / "dataset_loader.py", "code_loader").load_training_dataset(
        "coding:6", default_loader=None, load_dataset=None, load_from_disk=None)
    assert len(rows) == 6 and rows[1]["task"]["FAIL_TO_PASS"]
    agent = _load(ex / "run_agent.py", "code_agent")
    tools = sys.modules["coding_tools"]
    ws = tools.Workspace({"a.py": "x = 1\n"})
    try:
        assert ws.list_files() == {"files": ["a.py"]} and ws.read_file("a.py")["lines"] == ["1: x = 1"]
        assert "error" in ws.run_command("rm -rf .") and ws.rg("x =")["matches"] == ["a.py:1: x = 1"]
        try:
            ws.read_file("../../etc/passwd")
            raise AssertionError("path escape was allowed")
        except ValueError:
            pass
    finally:
        ws.close()
    task = rows[1]["task"]       # clamp: returns lo instead of hi

    def policy(messages):
        step = sum(1 for m in messages if m["role"] == "assistant")
        plan = [("read_file", {"path": "mod.py"}), ("run_command", {"command": task["test_command"]}),
                ("write_file", {"path": "mod.py", "content": task["reference_fix"]["mod.py"]}),
                ("submit", {"status": "solved", "summary": "fixed the upper bound"})]
        return _call(*plan[step])

    trajs = asyncio.run(agent.run_agent(ScriptedSession(policy), _batch([rows[1]])))
    turns = trajs[0].turns
    assert len(turns) == 4
    tool_msgs = [json.loads(m["content"]) for m in turns[-1].messages if m["role"] == "tool"]
    assert tool_msgs[1]["returncode"] != 0                       # the seeded bug fails its tests before the fix
    reward = _load(ex / "reward.py", "code_reward").reward_fn
    passed = [{"content": json.dumps(t)} for t in tool_msgs] + [{"content": json.dumps({"submitted": True, "tests_passed": True, "status": "solved"})}]
    assert reward(SimpleNamespace(tool_results=passed)) == 1.0
    failed = [{"content": json.dumps(t)} for t in tool_msgs] + [{"content": json.dumps({"submitted": True, "tests_passed": False, "status": "solved"})}]
    assert reward(SimpleNamespace(tool_results=failed)) == 0.1 and reward(SimpleNamespace(tool_results=[])) == 0.0


def test_tictactoe_one_step_task_and_web_ui():
    import threading
    import urllib.request
    from http.server import ThreadingHTTPServer

    base = ROOT / "examples" / "agentic" / "tictactoe"
    gen = _load(base / "dataset_generator.py", "ttt_gen")
    rows = gen.generate(60, seed=1)
    assert len(rows) == 60 and len({r["board"] for r in rows}) == 60
    assert sum(r["kind"] != "free" for r in rows) >= 35                       # mostly tactical positions
    for r in rows:
        assert r["board"].count("X") == r["board"].count("O") and all(r["board"][m - 1] == "." for m in r["answer"])
    loader = _load(base / "dataset_loader_no_tool.py", "ttt_loader")
    assert len(loader.load_training_dataset("tictactoe:16", default_loader=None, load_dataset=None, load_from_disk=None)) == 16

    reward = _load(base / "reward_no_tool.py", "ttt_reward")
    row = next(r for r in rows if r["kind"] == "win")
    good = row["answer"][0]
    other = next(i + 1 for i, c in enumerate(row["board"]) if c == "." and i + 1 not in row["answer"])
    taken = row["board"].index("X") + 1
    rec = lambda text: SimpleNamespace(completion=text, source_record=row, answer=row["answer"])   # noqa: E731
    assert reward.reward_fn(rec(f"I win with <move>{good}</move>")) == 1.0
    assert reward.reward_fn(rec(f"<move>{other}</move>")) == 0.2
    assert reward.reward_fn(rec(f"<move>{taken}</move>")) == 0.0 and reward.reward_fn(rec("no tag")) == 0.0

    agent = _load(base / "run_agent_no_tool.py", "ttt_agent")
    session = ScriptedSession(lambda messages: {"role": "assistant", "content": "<move>5</move>"})
    trajs = asyncio.run(agent.run_agent(session, _batch(rows[:4])))
    assert len(trajs) == 4 and session.calls == 4 and all(len(t.turns) == 1 for t in trajs)

    ui = _load(base / "web_ui.py", "ttt_ui")
    games = ui.Games(base_url=None)
    server = ThreadingHTTPServer(("127.0.0.1", 0), ui.make_handler(games))
    threading.Thread(target=server.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{server.server_address[1]}"

    def post(path, body):
        req = urllib.request.Request(url + path, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        return json.loads(urllib.request.urlopen(req, timeout=10).read())

    try:
        assert b"tic-tac-toe" in urllib.request.urlopen(url + "/", timeout=10).read()
        g = post("/api/new", {"human": "X"})
        assert g["board"] == "." * 9 and g["status"] == "playing"
        res = post("/api/move", {"id": g["id"], "cell": 4})
        assert res["board"][4] == "X" and res["board"].count("O") == 1 and res["reply"]["source"] == "rule opponent"
        assert "error" in post("/api/move", {"id": g["id"], "cell": 4})
        g2 = post("/api/new", {"human": "O"})
        assert g2["board"].count("X") == 1                                      # the other side opened
        for _ in range(6):                                                       # play the first free square to the end
            if res["status"] != "playing":
                break
            res = post("/api/move", {"id": g["id"], "cell": res["board"].index(".")})
        assert res["status"] in ("O wins", "X wins", "draw")
    finally:
        server.shutdown()


def test_coding_cli_applies_reference_fix_and_dataset_file_matches_generator(tmp_path):
    base = ROOT / "examples" / "agentic" / "coding"
    sys.modules.pop("agent_loop", None)
    cli = _load(base / "code_cli.py", "coding_cli")
    assert cli.main(["--reference-fix", "--task", "2"]) == 0            # known fix -> tests pass -> exit code 0
    out = tmp_path / "d.jsonl"
    assert cli.main(["--dump-dataset", str(out), "--n", "24"]) == 0
    assert out.read_text() == (base / "dataset.jsonl").read_text()      # the shipped file is the generator's output
    assert cli.main(["--reference-fix", "--dataset", str(out), "--task", "5"]) == 0


def test_duelgrid_web_ui_plays_full_turns():
    base = ROOT / "examples" / "agentic" / "duelgrid"
    ui = _load(base / "web_ui.py", "duel_ui")
    duels = ui.Duels(base_url=None)
    s = duels.new(seed=7)
    assert len(s["grid"]) == 6 and sum(row.count("A") + row.count("U") for row in s["grid"]) == 2 and s["outcome"] is None
    gid = s["id"]
    s2 = duels.act(gid, s["legal"][-1])
    assert s2["turn"] == 1 and s2["last"]["legal"] is True
    s3 = duels.act(gid, {"action": "teleport"})
    assert s3["turn"] == 2 and s3["last"]["legal"] is False               # an illegal answer costs the turn
    assert "error" in duels.model_move(gid) and "error" in duels.act("nope", {"action": "wait"})
    for _ in range(20):
        if s3["outcome"]:
            break
        s3 = duels.act(gid, {"action": "wait"})
    assert s3["outcome"] in ("win", "loss", "draw") and s3["legal"] == []
