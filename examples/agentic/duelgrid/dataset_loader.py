"""``--dataset-path duelgrid:N`` or a JSONL of start states written by ``dataset_generator.py``."""

from __future__ import annotations

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from game import new_state  # noqa: E402

PROMPT = ("You control A on a 6x6 grid and duel U. '+' heals, 'e' gives energy, 'x' is a trap. Attacks cost 1 energy and "
          "need an adjacent target. Reply with exactly one JSON action from the legal list.")


def load_training_dataset(dataset_path, *, default_loader, load_dataset, load_from_disk):
    path = str(dataset_path)
    if os.path.isfile(path):
        with open(path) as f:
            states = [json.loads(line) for line in f if line.strip()]
    else:
        try:
            n = int(path.rsplit(":", 1)[-1])
        except ValueError:
            n = 256
        states = [new_state(7000 + i) for i in range(n)]
    return [{"prompt": PROMPT, "answer": "win", "state": s} for s in states]
