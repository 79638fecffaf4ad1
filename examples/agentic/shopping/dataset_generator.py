"""Write shopping tasks as JSONL: ``python dataset_generator.py --output tasks.jsonl --count 2048 --seed 2026``."""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from game import make_task  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--output", required=True)
    ap.add_argument("--count", type=int, default=256)
    ap.add_argument("--seed", type=int, default=2026)
    args = ap.parse_args(argv)
    with open(args.output, "w") as f:
        for i in range(args.count):
            f.write(json.dumps(make_task(args.seed + i)) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
