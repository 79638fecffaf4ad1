"""Reference arm of bench.py: runs the unmodified reference installed under ``baseline/_ref``."""

from __future__ import annotations

import json


def run_reference(args) -> None:
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired up yet"}), flush=True)
