"""Score of the submitted bundle: 1.0 for a valid bundle reached through search -> inspect -> check ->
submit, 0.6 for a valid bundle by another route, partial credit for a submission that only breaks one rule."""

from __future__ import annotations

import json

EXPECTED = ["search_catalog", "inspect_items", "check_kit", "submit_bundle"]


def reward_fn(record) -> float:
    results = getattr(record, "tool_results", None) or []
    final = None
    for r in results:
        try:
            payload = json.loads(r.get("content") or "{}")
        except (ValueError, AttributeError):
            continue
        if isinstance(payload, dict) and "submitted" in payload:
            final = payload
    if final is None:
        return 0.0
    if final.get("ok"):
        used = final.get("tools_used") or []
        order = [t for t in used if t in EXPECTED]
        staged = all(t in order for t in EXPECTED) and order.index("check_kit") < order.index("submit_bundle")
        return 1.0 if staged else 0.6
    faults = len(final.get("missing") or []) + len(final.get("unmet") or []) + int(final.get("total", 0) > final.get("budget", 0))
    return 0.2 if faults == 1 else 0.0
