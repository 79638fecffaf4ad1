"""``--dataset-path shopping:N`` (or a JSONL written by ``dataset_generator.py``): one task per row."""

from __future__ import annotations

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from game import describe, make_task  # noqa: E402


def load_training_dataset(dataset_path, *, default_loader, load_dataset, load_from_disk):
    path = str(dataset_path)
    if os.path.isfile(path):
        with open(path) as f:
            tasks = [json.loads(line) for line in f if line.strip()]
    else:
        try:
            n = int(path.rsplit(":", 1)[-1])
        except ValueError:
            n = 256
        tasks = [make_task(2026 + i) for i in range(n)]
    return [{"prompt": describe(t), "answer": "ok", "task": t} for t in tasks]
