"""Watch or play DuelGrid in a browser.

    python examples/agentic/duelgrid/web_ui.py --port 8766                                   # you play A
    python examples/agentic/duelgrid/web_ui.py --port 8766 --base-url http://127.0.0.1:8000/v1   # the model can play A

Standard library only (``http.server``); the page is HTML + a little JavaScript and draws the grid as a table.
Routes (JSON):

    POST /api/new    {"seed": int | null}              -> state
    POST /api/act    {"id", "action": {...}}           -> state      (one full turn: A's action, then the scripted U)
    POST /api/model  {"id"}                            -> state      (ask the served model for A's action, then the turn)

``state`` = ``{"id", "grid": [[cell, ...], ...], "A": {...}, "U": {...}, "turn", "max_turns", "legal": [...],
"outcome": null | "win" | "loss" | "draw", "last": {"answer", "legal"}}``.  The model gets the same prompt as in
training (``run_agent.py``): the rendered map, both status lines and the list of legal actions.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import secrets
import sys
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from game import SIZE, legal_actions, new_state, outcome, render, step  # noqa: E402

PAGE = """<!doctype html>
<html><head><meta charset="utf-8"><title>DuelGrid</title>
<style>
body { font-family: sans-serif; margin: 2em; }
table { border-collapse: collapse; margin-bottom: 1em; }
td { width: 44px; height: 44px; border: 1px solid #888; text-align: center; font-size: 22px; }
td.A { background: #cde; font-weight: bold; } td.U { background: #ecc; font-weight: bold; }
button { margin: 2px; }
#last { color: #444; white-space: pre-wrap; }
</style></head><body>
<h2>DuelGrid</h2>
<p><button onclick="newGame()">new game</button> <button id="ask" onclick="askModel()">let the model move</button>
<span id="status"></span></p>
<table id="grid"></table>
<div id="bars"></div>
<div id="actions"></div>
<div id="last"></div>
<p>Legend: A you / the policy, U scripted opponent, + health, e energy, x trap.</p>
<script>
let gid = null;
async function post(path, body) {
  const r = await fetch(path, {method: 'POST', headers: {'Content-Type': 'application/json'}, body: JSON.stringify(body)});
  return r.json();
}
function show(s) {
  if (s.error) { alert(s.error); return; }
  gid = s.id;
  const t = document.getElementById('grid'); t.innerHTML = '';
  for (const row of s.grid) { const tr = t.insertRow(); for (const cell of row) { const td = tr.insertCell();
    td.textContent = cell === '.' ? '' : cell; if (cell === 'A' || cell === 'U') td.className = cell; } }
  document.getElementById('bars').textContent =
      'A hp ' + s.A.hp + ' en ' + s.A.en + '   |   U hp ' + s.U.hp + ' en ' + s.U.en + '   |   turn ' + s.turn + '/' + s.max_turns;
  document.getElementById('status').textContent = s.outcome ? 'result: ' + s.outcome : '';
  const a = document.getElementById('actions'); a.innerHTML = '';
  if (!s.outcome) for (const act of s.legal) { const b = document.createElement('button');
    b.textContent = act.action + (act.dir ? ' ' + act.dir : ''); b.onclick = () => doAct(act); a.appendChild(b); }
  document.getElementById('last').textContent = s.last ? 'last answer: ' + s.last.answer + (s.last.legal ? '' : '   (illegal: counted as wait)') : '';
}
async function newGame() { show(await post('/api/new', {})); }
async function doAct(act) { show(await post('/api/act', {id: gid, action: act})); }
async function askModel() { show(await post('/api/model', {id: gid})); }
newGame();
</script></body></html>
"""

SYSTEM_PROMPT = ("You control unit A in a grid duel against unit U. Answer with exactly one JSON object taken from the "
                 "list of legal actions, and nothing else.")


def view(gid: str, s: dict, last: dict | None = None) -> dict:
    grid = []
    for r in range(SIZE):
        row = []
        for c in range(SIZE):
            row.append("A" if s["A"]["pos"] == [r, c] else "U" if s["U"]["pos"] == [r, c] else s["tiles"].get(f"{r},{c}", "."))
        grid.append(row)
    return {"id": gid, "grid": grid, "A": s["A"], "U": s["U"], "turn": s["turn"], "max_turns": s["max_turns"],
            "legal": legal_actions(s, "A") if outcome(s) is None else [], "outcome": outcome(s), "last": last}


class Duels:
    def __init__(self, base_url: str | None = None, model: str = "policy", timeout_s: float = 60.0):
        self.base_url, self.model, self.timeout_s = base_url, model, timeout_s
        self.states: dict[str, dict] = {}

    def new(self, seed=None) -> dict:
        gid = secrets.token_hex(8)
        self.states[gid] = new_state(int(seed) if seed is not None else random.randrange(1 << 30))
        if len(self.states) > 1024:
            for key in list(self.states)[:256]:
                self.states.pop(key, None)
        return view(gid, self.states[gid])

    def _turn(self, gid: str, answer: str) -> dict:
        s = self.states.get(gid)
        if s is None:
            return {"error": "unknown game"}
        if outcome(s) is not None:
            return {"error": "the game is over"}
        s, legal = step(s, answer)
        self.states[gid] = s
        return view(gid, s, {"answer": answer, "legal": legal})

    def act(self, gid: str, action) -> dict:
        return self._turn(gid, json.dumps(action if isinstance(action, dict) else {"action": "invalid"}))

    def model_move(self, gid: str) -> dict:
        s = self.states.get(gid)
        if s is None:
            return {"error": "unknown game"}
        if not self.base_url:
            return {"error": "no --base-url was given: there is no model to ask"}
        prompt = f"{render(s)}\n\nLegal actions:\n" + "\n".join(json.dumps(a) for a in legal_actions(s, "A"))
        body = {"model": self.model, "messages": [{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": prompt}]}
        req = urllib.request.Request(self.base_url.rstrip("/") + "/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json", "Authorization": "Bearer none"})
        try:
            with urllib.request.urlopen(req, timeout=self.timeout_s) as resp:
                answer = json.loads(resp.read())["choices"][0]["message"].get("content") or ""
        except Exception as exc:  # noqa: BLE001
            return {"error": f"endpoint error: {exc}"}
        return self._turn(gid, answer)


def make_handler(duels: Duels):
    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *args):
            return

        def _send(self, code: int, body: bytes, ctype: str):
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path in ("/", "/index.html"):
                self._send(200, PAGE.encode(), "text/html; charset=utf-8")
            else:
                self._send(404, b"not found", "text/plain")

        def do_POST(self):
            try:
                n = int(self.headers.get("Content-Length") or 0)
                body = json.loads(self.rfile.read(n) or b"{}")
            except ValueError:
                return self._send(400, b'{"error": "bad json"}', "application/json")
            if self.path == "/api/new":
                out = duels.new(body.get("seed"))
            elif self.path == "/api/act":
                out = duels.act(str(body.get("id")), body.get("action"))
            elif self.path == "/api/model":
                out = duels.model_move(str(body.get("id")))
            else:
                return self._send(404, b'{"error": "not found"}', "application/json")
            self._send(200, json.dumps(out).encode(), "application/json")

    return Handler


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8766)
    ap.add_argument("--base-url", default=None)
    ap.add_argument("--model", default="policy")
    args = ap.parse_args(argv)
    server = ThreadingHTTPServer((args.host, args.port), make_handler(Duels(args.base_url, args.model)))
    print(f"open http://{args.host}:{args.port}/")
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
