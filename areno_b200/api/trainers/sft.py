"""Supervised fine-tuning: ``prompt`` / ``response`` rows -> masked ``TrainSequence`` -> next-token NLL on
the response tokens (``areno/api/trainers/sft.py:29-177`` in the reference).  Rows that are empty,
all-prompt, or over the prompt / response token budgets are skipped; a dataset that yields no
row at all is an error."""

from __future__ import annotations

from typing import Any

from ..data_utils import prompt_response_to_tokens_and_mask
from ..models import TrainSequence
from .offline import OfflineTrainer


def record_to_train_sequence(record: Any, tokenizer, *, max_prompt_tokens: int, max_new_tokens: int):
    record = dict(record)
    if "prompt" not in record or "response" not in record:
        raise ValueError("SFT dataset loader must return rows with `prompt` and `response`; "
                         "normalize raw dataset fields in --dataset-loader-fn")
    if record["prompt"] is None or record["response"] is None or not str(record["response"]):
        return None
    eos = tokenizer.eos_token_id if tokenizer.eos_token_id is not None else 0
    tokens, mask = prompt_response_to_tokens_and_mask(str(record["prompt"]), str(record["response"]), tokenizer, eos)
    if len(tokens) < 2:
        return None
    n_prompt, n_resp = mask.count(True), mask[1:].count(False)
    if n_prompt > max_prompt_tokens or n_resp > max_new_tokens or n_resp == 0:
        return None
    zeros = [0.0] * len(tokens)
    return TrainSequence(prompt_mask=mask, tokens=tokens, logprobs=zeros, advantages=zeros, eos_token_id=eos)


class SFTTrainer(OfflineTrainer):
    unit = "rows"

    def _iter_train_batches(self, tokenizer):
        batch, skipped, accepted = [], 0, 0
        total = len(self.dataset)
        for i in range(total):
            seq = record_to_train_sequence(self.dataset[i], tokenizer, max_prompt_tokens=self.config.max_prompt_tokens,
                                           max_new_tokens=self.config.max_new_tokens)
            if seq is None:
                skipped += 1
                continue
            accepted += 1
            batch.append(seq)
            if len(batch) >= self.config.batch_size:
                yield batch
                batch = []
        if skipped:
            self.logger.info("stage=sft_dataset_filter skipped_long_or_empty=%d", skipped)
        if accepted == 0:
            raise ValueError(
                "SFT dataset produced no valid training rows after filtering: "
                f"scanned {total} row(s), skipped {skipped} as empty, over-budget, or all-prompt examples. "
                "Check dataset quality, --max-prompt-tokens, and --max-new-tokens.")
        if batch:
            yield batch


__all__ = ["SFTTrainer", "record_to_train_sequence"]
