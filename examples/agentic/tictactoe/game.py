"""Tic-tac-toe rules and a fixed-policy opponent (win if possible, else block, else first free)."""

from __future__ import annotations

LINES = [(0, 1, 2), (3, 4, 5), (6, 7, 8), (0, 3, 6), (1, 4, 7), (2, 5, 8), (0, 4, 8), (2, 4, 6)]


def winner(board: list[str]) -> str | None:
    for a, b, c in LINES:
        if board[a] != "." and board[a] == board[b] == board[c]:
            return board[a]
    return "draw" if "." not in board else None


def render(board: list[str]) -> str:
    return "\n".join(" ".join(board[r * 3:r * 3 + 3]) for r in range(3))


def opponent_move(board: list[str], me: str = "O", other: str = "X") -> int:
    for mark in (me, other):
        for a, b, c in LINES:
            cells = [board[a], board[b], board[c]]
            if cells.count(mark) == 2 and cells.count(".") == 1:
                return (a, b, c)[cells.index(".")]
    return board.index(".")
