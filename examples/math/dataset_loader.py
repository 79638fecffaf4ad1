"""GSM8K-style rows -> ``{"prompt", "answer"}`` for ``areno train --dataset-loader-fn``.

    areno train --algo grpo --ckpt <model> --dataset-path openai/gsm8k \
        --dataset-loader-fn examples/math/dataset_loader.py --reward-fn-path examples/math/reward.py
"""

from __future__ import annotations

SYSTEM = "Solve the problem step by step and give the final answer after '####'."


def _final_answer(solution: str) -> str:
    tail = solution.rsplit("####", 1)[-1] if "####" in solution else solution
    return tail.strip().replace(",", "")


def load_training_dataset(dataset_path, *, default_loader, load_dataset, load_from_disk):
    rows = default_loader(dataset_path)
    out = []
    for row in rows:
        question = row.get("question") or row.get("problem") or row.get("prompt")
        solution = row.get("answer") or row.get("solution") or ""
        if not question:
            continue
        out.append({"prompt": f"{SYSTEM}\n\n{question}", "answer": _final_answer(str(solution))})
    return out
