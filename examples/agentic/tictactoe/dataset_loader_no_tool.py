"""Loader of the one-step task: a JSONL file written by ``dataset_generator.py``, or ``tictactoe:<n>`` to
generate ``n`` positions in memory (seed 0)."""

from __future__ import annotations

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dataset_generator import generate  # noqa: E402


def load_training_dataset(dataset_path, *, default_loader, load_dataset, load_from_disk):
    path = str(dataset_path)
    if os.path.isfile(path):
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]
    try:
        n = int(path.rsplit(":", 1)[-1])
    except ValueError:
        n = 512
    return generate(n, seed=0)
