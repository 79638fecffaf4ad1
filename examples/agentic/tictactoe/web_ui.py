"""Play tic-tac-toe in a browser against a served policy (or the rule opponent).

    python examples/agentic/tictactoe/web_ui.py --port 8765 --base-url http://127.0.0.1:8000/v1

The page is plain HTML + a few lines of JavaScript served by the standard library's ``http.server``; the server
keeps one board per browser tab (a random game id) and exposes two JSON routes:

    POST /api/new   {"human": "X" | "O"}            -> {"id", "board", "status"}
    POST /api/move  {"id", "cell"}                   -> {"board", "status", "reply": {"cell", "raw"}}

The side that is not the human is played by the model behind ``--base-url`` (an OpenAI-compatible
``/chat/completions`` endpoint such as ``areno serve``) with the one-step prompt of ``run_agent_no_tool.py``; without
``--base-url``, or when the model's answer is not a legal move, the rule opponent of ``game.py`` moves instead and the
reply says so.
"""

from __future__ import annotations

import argparse
import json
import os
import secrets
import sys
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from game import labelled, legal_moves, opponent_move, winner  # noqa: E402
from reward_no_tool import parse_move  # noqa: E402

PAGE = """<!doctype html>
<html><head><meta charset="utf-8"><title>tic-tac-toe</title>
<style>
body { font-family: sans-serif; margin: 2em; }
table { border-collapse: collapse; }
td { width: 72px; height: 72px; border: 2px solid #444; text-align: center; font-size: 40px; cursor: pointer; }
td.taken { cursor: default; }
#log { margin-top: 1em; white-space: pre-wrap; color: #333; max-width: 40em; }
</style></head><body>
<h2>tic-tac-toe</h2>
<p>You play <select id="side"><option>X</option><option>O</option></select>
<button onclick="newGame()">new game</button> <span id="status"></span></p>
<table id="grid"></table>
<div id="log"></div>
<script>
let game = null;
function draw(board) {
  const t = document.getElementById('grid'); t.innerHTML = '';
  for (let r = 0; r < 3; r++) { const tr = t.insertRow();
    for (let c = 0; c < 3; c++) { const i = r * 3 + c; const td = tr.insertCell();
      td.textContent = board[i] === '.' ? '' : board[i];
      if (board[i] !== '.') td.className = 'taken'; else td.onclick = () => move(i); } }
}
async function post(path, body) {
  const r = await fetch(path, {method: 'POST', headers: {'Content-Type': 'application/json'}, body: JSON.stringify(body)});
  return r.json();
}
function show(res) {
  draw(res.board); document.getElementById('status').textContent = res.status;
  if (res.reply) document.getElementById('log').textContent =
      'opponent played ' + (res.reply.cell + 1) + ' (' + res.reply.source + ')\\n' + (res.reply.raw || '');
}
async function newGame() { const res = await post('/api/new', {human: document.getElementById('side').value}); game = res.id; show(res); }
async function move(i) { if (!game) return; const res = await post('/api/move', {id: game, cell: i}); if (res.error) alert(res.error); else show(res); }
newGame();
</script></body></html>
"""

SYSTEM_PROMPT = ("You are a careful tic-tac-toe player and you play {me}. Numbers on the board are free squares, not "
                 "marks. Take a win if there is one; otherwise stop {other} from completing a row; otherwise pick any "
                 "free square. Reply with exactly one tag such as <move>5</move>.")


def status_of(board: list[str]) -> str:
    w = winner(board)
    return "playing" if w is None else "draw" if w == "draw" else f"{w} wins"


class Games:
    """Boards by game id, and the non-human side's move."""

    def __init__(self, base_url: str | None = None, model: str = "policy", api_key: str = "none", timeout_s: float = 60.0):
        self.base_url, self.model, self.api_key, self.timeout_s = base_url, model, api_key, timeout_s
        self.boards: dict[str, tuple[list[str], str]] = {}   # id -> (board, human mark)

    # ---------------------------------------------------------------- model
    def ask_model(self, board: list[str], me: str) -> tuple[int | None, str]:
        """The model's move (0-based) and its raw answer; ``None`` when there is no endpoint or no legal move in it."""
        if not self.base_url:
            return None, ""
        other = "O" if me == "X" else "X"
        body = {"model": self.model, "messages": [
            {"role": "system", "content": SYSTEM_PROMPT.format(me=me, other=other)},
            {"role": "user", "content": f"You play {me} and it is your move.\n\n{labelled(board)}"}]}
        req = urllib.request.Request(self.base_url.rstrip("/") + "/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json", "Authorization": f"Bearer {self.api_key}"})
        try:
            with urllib.request.urlopen(req, timeout=self.timeout_s) as resp:
                raw = json.loads(resp.read())["choices"][0]["message"].get("content") or ""
        except Exception as exc:  # noqa: BLE001 - a dead endpoint must not end the game
            return None, f"endpoint error: {exc}"
        move = parse_move(raw)
        if move is None or board[move - 1] != ".":
            return None, raw
        return move - 1, raw

    def reply(self, board: list[str], me: str) -> dict:
        cell, raw = self.ask_model(board, me)
        source = "model"
        if cell is None:
            other = "O" if me == "X" else "X"
            cell, source = opponent_move(board, me=me, other=other), "rule opponent"
        board[cell] = me
        return {"cell": cell, "raw": raw, "source": source}

    # ---------------------------------------------------------------- routes
    def new(self, human: str) -> dict:
        human = "O" if str(human).upper() == "O" else "X"
        gid = secrets.token_hex(8)
        board = ["."] * 9
        out = {"id": gid}
        if human == "O":                 # X moves first
            out["reply"] = self.reply(board, "X")
        self.boards[gid] = (board, human)
        if len(self.boards) > 1024:      # forget the oldest games
            for key in list(self.boards)[:256]:
                self.boards.pop(key, None)
        out.update(board="".join(board), status=status_of(board))
        return out

    def move(self, gid: str, cell: int) -> dict:
        if gid not in self.boards:
            return {"error": "unknown game"}
        board, human = self.boards[gid]
        if winner(board) is not None:
            return {"error": "the game is over"}
        if not isinstance(cell, int) or cell not in legal_moves(board):
            return {"error": "that square is taken"}
        board[cell] = human
        out = {}
        if winner(board) is None:
            out["reply"] = self.reply(board, "O" if human == "X" else "X")
        out.update(board="".join(board), status=status_of(board))
        return out


def make_handler(games: Games):
    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *args):   # quiet
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
                out = games.new(body.get("human", "X"))
            elif self.path == "/api/move":
                out = games.move(str(body.get("id")), body.get("cell"))
            else:
                return self._send(404, b'{"error": "not found"}', "application/json")
            self._send(200, json.dumps(out).encode(), "application/json")

    return Handler


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8765)
    ap.add_argument("--base-url", default=None, help="OpenAI-compatible endpoint of the policy, e.g. http://127.0.0.1:8000/v1")
    ap.add_argument("--model", default="policy")
    args = ap.parse_args(argv)
    server = ThreadingHTTPServer((args.host, args.port), make_handler(Games(args.base_url, args.model)))
    print(f"open http://{args.host}:{args.port}/  (opponent: {'model at ' + args.base_url if args.base_url else 'rule opponent'})")
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
