"""Game outcome reward read from the last tool result: win 1.0, draw 0.3, anything else 0."""

from __future__ import annotations

import json


def reward_fn(record) -> float:
    results = getattr(record, "tool_results", None) or []
    if not results:
        return 0.0
    try:
        outcome = json.loads(results[-1].get("content") or "{}").get("result")
    except (ValueError, AttributeError):
        return 0.0
    return {"win": 1.0, "draw": 0.3}.get(outcome, 0.0)
