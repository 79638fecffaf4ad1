"""Outcome reward with shaping, recomputed by replaying the episode from the recorded answers (the rule engine
and the opponent are deterministic): win 1.0, draw 0.4, loss 0; plus up to 0.3 for damage dealt, minus 0.05
per illegal answer (floored at 0)."""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import game  # noqa: E402


def reward_fn(record) -> float:
    start = (getattr(record, "source_record", None) or {}).get("state")
    if not start:
        return 0.0
    answers = [m.get("content") or "" for m in (getattr(record, "messages", None) or []) if m.get("role") == "assistant"]
    final = game.replay(start, answers)
    if final["outcome"] is None:
        return 0.0   # the episode was cut short
    base = {"win": 1.0, "draw": 0.4}.get(final["outcome"], 0.0)
    shaped = base + 0.3 * max(0, 6 - final["enemy_hp"]) / 6.0 - 0.05 * final["illegal"]
    return float(max(0.0, min(1.3, shaped)))
