"""Synthetic prompts: each row is one game to play as X from the empty board (seeded opening for O)."""

from __future__ import annotations

import random


def load_training_dataset(dataset_path, *, default_loader, load_dataset, load_from_disk):
    rng = random.Random(0)
    n = 256
    try:
        n = int(str(dataset_path).rsplit(":", 1)[-1])
    except ValueError:
        pass
    return [{"prompt": "Play tic-tac-toe as X. Use the place_mark tool to move.", "answer": "win", "seed": rng.randrange(1 << 30)}
            for _ in range(n)]
