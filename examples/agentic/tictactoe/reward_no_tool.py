"""Reward of the one-step task: 1.0 for a move a careful player accepts (win > block > any free square), 0.2 for
another legal move, 0 for an illegal or unparsable answer.  The answer is the last ``<move>N</move>`` tag."""

from __future__ import annotations

import re

_TAG = re.compile(r"<move>\s*([1-9])\s*</move>")


def parse_move(text: str) -> int | None:
    found = _TAG.findall(text or "")
    return int(found[-1]) if found else None


def reward_fn(record) -> float:
    row = getattr(record, "source_record", None) or {}
    move = parse_move(getattr(record, "completion", "") or "")
    if move is None:
        return 0.0
    board = str(row.get("board", ""))
    if len(board) != 9 or board[move - 1] != ".":
        return 0.0
    accepted = getattr(record, "answer", None) or row.get("answer") or []
    return 1.0 if move in set(accepted) else 0.2
