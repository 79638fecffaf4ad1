"""Alpaca rows -> ``{"prompt", "response"}`` for ``areno train --algo sft``.

    areno train --algo sft --ckpt <model> --dataset-path tatsu-lab/alpaca \
        --dataset-loader-fn examples/sft/alpaca/dataset_loader.py
"""

from __future__ import annotations


def load_training_dataset(dataset_path, *, default_loader, load_dataset, load_from_disk):
    out = []
    for row in default_loader(dataset_path):
        instruction = (row.get("instruction") or "").strip()
        extra = (row.get("input") or "").strip()
        response = (row.get("output") or row.get("response") or "").strip()
        if not instruction or not response:
            continue
        prompt = f"{instruction}\n\n{extra}" if extra else instruction
        out.append({"prompt": prompt, "response": response})
    return out
