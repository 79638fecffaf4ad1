"""Write a JSONL file of one-step tic-tac-toe positions (X to move) for the no-tool task.

    python examples/agentic/tictactoe/dataset_generator.py --out /tmp/ttt.jsonl --n 2000 --seed 0

Each row: ``{"prompt": <board with numbered free cells>, "board": "X.O...", "answer": [cells a careful player
accepts, 1-based], "kind": "win" | "block" | "free"}``.  Positions are unique within a file.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from game import completing_moves, good_moves, labelled, random_position  # noqa: E402


def make_row(board: list[str]) -> dict:
    kind = "win" if completing_moves(board, "X") else "block" if completing_moves(board, "O") else "free"
    prompt = ("You play X and it is your move. Free squares show their number.\n\n" + labelled(board) +
              "\n\nAnswer with one tag such as <move>5</move>.")
    return {"prompt": prompt, "board": "".join(board), "answer": [m + 1 for m in good_moves(board)], "kind": kind}


def generate(n: int, seed: int = 0, tactical_share: float = 0.7) -> list[dict]:
    """``tactical_share`` of the rows have a win or a block on the board (the rest are free choices)."""
    rng = random.Random(seed)
    rows, seen = [], set()
    attempts = 0
    while len(rows) < n and attempts < 200 * n:
        attempts += 1
        board = random_position(rng)
        key = "".join(board)
        if key in seen:
            continue
        row = make_row(board)
        want_tactical = len([r for r in rows if r["kind"] != "free"]) < tactical_share * (len(rows) + 1)
        if want_tactical and row["kind"] == "free":
            continue
        seen.add(key)
        rows.append(row)
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--out", required=True)
    ap.add_argument("--n", type=int, default=2000)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    rows = generate(args.n, args.seed)
    with open(args.out, "w") as f:
        for row in rows:
            f.write(json.dumps(row) + "\n")
    print(f"wrote {len(rows)} positions to {args.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
