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


# ------------------------------------------------------------------ one-step ("no tool") task helpers
def legal_moves(board: list[str]) -> list[int]:
    return [i for i, c in enumerate(board) if c == "."]


def completing_moves(board: list[str], mark: str) -> list[int]:
    """Free cells that give ``mark`` three in a row at once."""
    out = []
    for a, b, c in LINES:
        cells = [board[a], board[b], board[c]]
        if cells.count(mark) == 2 and cells.count(".") == 1:
            out.append((a, b, c)[cells.index(".")])
    return sorted(set(out))


def good_moves(board: list[str]) -> list[int]:
    """The moves a careful X player accepts: a win if there is one, else a block of O's threat, else any free cell."""
    return completing_moves(board, "X") or completing_moves(board, "O") or legal_moves(board)


def labelled(board: list[str]) -> str:
    """Board with the free cells shown as their numbers 1-9 (marks are X / O), three rows."""
    cells = [c if c != "." else str(i + 1) for i, c in enumerate(board)]
    return "\n".join(" | ".join(cells[r * 3:r * 3 + 3]) for r in range(3))


def random_position(rng, min_marks: int = 2, max_marks: int = 6) -> list[str]:
    """A reachable position with X to move and no winner yet: marks are placed alternately, O first or X first so
    that the counts allow X the next move."""
    while True:
        n = rng.randrange(min_marks, max_marks + 1)
        n -= n % 2                     # X moves when both sides have played equally often
        board = ["."] * 9
        cells = list(range(9))
        rng.shuffle(cells)
        for j, cell in enumerate(cells[:n]):
            board[cell] = "X" if j % 2 == 0 else "O"
        if winner(board) is None:
            return board
