"""``--dataset-path coding:N`` (generated tasks) or a JSONL of task records."""

from __future__ import annotations

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from tasks import make_task  # noqa: E402


def load_training_dataset(dataset_path, *, default_loader, load_dataset, load_from_disk):
    path = str(dataset_path)
    if os.path.isfile(path):
        with open(path) as f:
            tasks = [json.loads(line) for line in f if line.strip()]
    else:
        try:
            n = int(path.rsplit(":", 1)[-1])
        except ValueError:
            n = 100
        tasks = [make_task(i) for i in range(n)]
    return [{"prompt": ("Fix the bug described below in the repository. Inspect files, edit them, run the tests and then call "
                        f"submit.\n\nIssue: {t['problem_statement']}"), "answer": "solved", "task": t} for t in tasks]
