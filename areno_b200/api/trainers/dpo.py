"""Direct preference optimisation with one frozen reference role.

Rows are ``{prompt, chosen, rejected}`` (text) or ``{chosen, rejected}`` as chat-message lists whose
common token prefix is the prompt.  Every pair becomes two adjacent ``TrainSequence`` rows
(chosen first), so ``mini_bs`` must be even.  Before each update the reference role scores the
batch and fills ``ref_logprobs`` (``areno/api/trainers/dpo.py:27-212`` in the reference)."""

from __future__ import annotations

import time
from functools import partial
from typing import Any

from ..agentic import common_prefix_len
from ..data_utils import apply_chat_template, encode_prompt_value, response_to_tokens_and_mask
from ..models import TrainSequence
from ..roles import ModelRole
from .offline import OfflineTrainer


def _sequence(tokens, mask, eos, max_seq_len):
    if len(tokens) < 2 or len(tokens) > max_seq_len or not any(not m for m in mask[1:]):
        return None
    zeros = [0.0] * len(tokens)
    return TrainSequence(prompt_mask=mask, tokens=tokens, logprobs=zeros, advantages=zeros, eos_token_id=eos)


def record_to_train_pair(record: Any, tokenizer, *, max_seq_len: int):
    record = dict(record)
    eos = tokenizer.eos_token_id if tokenizer.eos_token_id is not None else 0
    if "chosen" not in record or "rejected" not in record:
        raise ValueError("DPO dataset row must contain `chosen` and `rejected`")
    chosen, rejected = record["chosen"], record["rejected"]
    if isinstance(chosen, list) and isinstance(rejected, list):
        c_tok, r_tok = apply_chat_template(tokenizer, chosen), apply_chat_template(tokenizer, rejected)
        n = common_prefix_len(c_tok, r_tok)
        c_mask = [True] * n + [False] * (len(c_tok) - n)
        r_mask = [True] * n + [False] * (len(r_tok) - n)
    else:
        if "prompt" not in record:
            raise ValueError("DPO prompt/response rows must contain `prompt`")
        prompt_ids = encode_prompt_value(tokenizer, record["prompt"])
        c_tok, c_mask = response_to_tokens_and_mask(prompt_ids, str(chosen), tokenizer, eos)
        r_tok, r_mask = response_to_tokens_and_mask(prompt_ids, str(rejected), tokenizer, eos)
    a, b = _sequence(c_tok, c_mask, eos, max_seq_len), _sequence(r_tok, r_mask, eos, max_seq_len)
    return None if a is None or b is None else [a, b]


class DPOTrainer(OfflineTrainer):
    unit = "pairs"

    def __init__(self, config, *, instance, dataset, reward_fn=None, loss_fn=None):
        if int(config.mini_bs) % 2 != 0:
            raise ValueError("DPO requires --mini-bs to be even so chosen/rejected pairs stay together")
        super().__init__(config, instance=instance, dataset=dataset, reward_fn=None,
                         loss_fn=partial(loss_fn, beta=config.dpo_beta))
        self.roles = {"ref": ModelRole("ref", config.ref_ckpt or config.ckpt, trainable=False)}

    def _prepare(self) -> None:
        for role in self.roles.values():
            self.logger.info("role=%s stage=init_start trainable=%s path=%s", role.name, role.trainable, role.path)
        self.areno.ensure_roles(self.roles)
        for role in self.roles.values():
            self.logger.info("role=%s stage=init_end trainable=%s", role.name, role.trainable)

    def _count(self, train_batch) -> int:
        return len(train_batch) // 2

    def _iter_train_batches(self, tokenizer):
        max_seq_len = self.config.max_prompt_tokens + self.config.max_new_tokens
        batch, skipped = [], 0
        for i in range(len(self.dataset)):
            pair = record_to_train_pair(self.dataset[i], tokenizer, max_seq_len=max_seq_len)
            if pair is None:
                skipped += 1
                continue
            batch.extend(pair)
            if len(batch) >= self.config.batch_size * 2:
                yield batch
                batch = []
        if skipped:
            self.logger.info("stage=dpo_dataset_filter skipped_invalid_or_long=%d", skipped)
        if batch:
            yield batch

    def _before_train(self, train_batch, epoch: int, step: int) -> dict:
        self.logger.info("epoch=%d step=%d role=ref stage=logprob_score_start rows=%d", epoch, step, len(train_batch))
        t0 = time.perf_counter()
        rows = self.areno.score_logprobs("ref", [s.tokens for s in train_batch])
        dt = time.perf_counter() - t0
        self.logger.info("epoch=%d step=%d role=ref stage=logprob_score_end rows=%d", epoch, step, len(train_batch))
        for seq, ref in zip(train_batch, rows):
            if len(ref) != len(seq.tokens):
                raise ValueError("reference role returned misaligned logprobs")
            seq.ref_logprobs = [float(v) for v in ref]
            seq.values = [0.0] * len(seq.tokens)
            seq.returns = [0.0] * len(seq.tokens)
        return {"ref_logprob_forward_time_s": dt}


__all__ = ["DPOTrainer", "record_to_train_pair"]
