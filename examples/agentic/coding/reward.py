"""1.0 when ``submit`` ran the task's tests and they passed, 0.1 for a submission with failing tests that at
least ran the tests earlier, 0 otherwise."""

from __future__ import annotations

import json


def reward_fn(record) -> float:
    results = getattr(record, "tool_results", None) or []
    submitted, ran_tests = None, False
    for r in results:
        try:
            payload = json.loads(r.get("content") or "{}")
        except (ValueError, AttributeError):
            continue
        if not isinstance(payload, dict):
            continue
        if payload.get("submitted"):
            submitted = payload
        elif "returncode" in payload:
            ran_tests = True
    if submitted is None:
        return 0.0
    if submitted.get("tests_passed") and submitted.get("status") == "solved":
        return 1.0
    return 0.1 if ran_tests else 0.0
