"""Dataset rows of the offline trainers (SFT, DPO) and the tokenizer helpers they share, on the CPU: prompt / response
masks, token budgets, rows that are dropped, preference pairs from text and from chat messages, EOS ids from tokenizer
and ``config.json``, the ``enable_thinking`` switch of chat templates, and the defaults of the SDK's data models.
Behaviours follow the reference's ``tests/test_trainer_dataset_utils_cpu.py`` and ``tests/test_tokenizer_api_cpu.py``."""

from __future__ import annotations

import json
import logging
from types import SimpleNamespace

import pytest

from areno_b200.api.data_utils import (apply_chat_template, encode_prompt_value, first_text, first_value, has_any,
                                       prompt_response_to_tokens_and_mask, response_to_tokens_and_mask)
from areno_b200.api.models import RolloutResult, RolloutSequence, SamplingParams, TrainSequence
from areno_b200.api.tokenizer import (apply_chat_template_with_options, configure_chat_template_enable_thinking,
                                      encode_generation_prompt, eos_token_ids, looks_chat_formatted, normalize_token_ids)
from areno_b200.api.trainers.dpo import DPOTrainer, record_to_train_pair
from areno_b200.api.trainers.sft import SFTTrainer, record_to_train_sequence
from tests.helpers import FakeTokenizer


class TemplateTokenizer(FakeTokenizer):
    """Chat template ``[role] content`` per message plus ``[assistant]`` as generation prompt; records its calls."""

    chat_template = "[role] content"

    def __init__(self, accepts_thinking=True):
        super().__init__()
        self.accepts_thinking = accepts_thinking
        self.calls: list[dict] = []

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, **kw):
        if "enable_thinking" in kw and not self.accepts_thinking:
            raise TypeError("apply_chat_template() got an unexpected keyword argument 'enable_thinking'")
        self.calls.append(dict(kw, gen=add_generation_prompt))
        words = []
        for m in messages:
            words += [f"[{m['role']}]", m["content"]]
        if add_generation_prompt:
            words.append("[assistant]")
        if kw.get("enable_thinking") is False:
            words.append("[nothink]")
        text = " ".join(words)
        return self.encode(text) if tokenize else text


# -------------------------------------------------------------------------------------------------- SFT rows

def test_sft_row_masks_the_prompt_and_appends_eos():
    tok = FakeTokenizer()
    seq = record_to_train_sequence({"prompt": "say hello", "response": "hello there friend", "extra": 1}, tok,
                                   max_prompt_tokens=8, max_new_tokens=8)
    n_p = len(tok.encode("say hello"))
    assert seq.tokens[:n_p] == tok.encode("say hello") and seq.tokens[-1] == tok.eos_token_id
    assert seq.tokens[n_p:-1] == tok.encode("hello there friend")
    assert seq.prompt_mask == [True] * n_p + [False] * 4
    assert seq.logprobs == [0.0] * len(seq.tokens) and seq.advantages == [0.0] * len(seq.tokens)
    assert seq.eos_token_id == tok.eos_token_id


def test_sft_does_not_double_an_eos_that_the_response_already_ends_with():
    tok = FakeTokenizer()
    toks, mask = response_to_tokens_and_mask([5, 6], "word", tok, eos_token_id=tok.encode("word")[-1])
    assert toks == [5, 6] + tok.encode("word") and mask == [True, True, False]
    toks, _ = response_to_tokens_and_mask([5], "word", tok, eos_token_id=None)
    assert toks == [5] + tok.encode("word")


def test_sft_wants_rows_that_the_loader_normalised():
    with pytest.raises(ValueError, match="`prompt` and `response`"):
        record_to_train_sequence({"instruction": "x", "output": "y"}, FakeTokenizer(), max_prompt_tokens=8, max_new_tokens=8)


@pytest.mark.parametrize("row", [
    {"prompt": "p", "response": ""}, {"prompt": None, "response": "r"}, {"prompt": "p", "response": None},
])
def test_sft_drops_rows_without_a_target(row):
    assert record_to_train_sequence(row, FakeTokenizer(), max_prompt_tokens=8, max_new_tokens=8) is None


def test_sft_budgets_apply_to_prompt_and_response_separately():
    tok = FakeTokenizer()
    row = {"prompt": "one two three", "response": "a b c d"}                # 3 prompt tokens, 4 + EOS response tokens
    assert record_to_train_sequence(row, tok, max_prompt_tokens=3, max_new_tokens=5) is not None
    assert record_to_train_sequence(row, tok, max_prompt_tokens=2, max_new_tokens=50) is None
    assert record_to_train_sequence(row, tok, max_prompt_tokens=50, max_new_tokens=4) is None


class _Areno:
    def __init__(self, tok):
        self.tok, self.batches = tok, []

    def get_tokenizer(self):
        return self.tok

    def train(self, batch, loss_fn, mini_bs, gradient_accumulation_steps):
        self.batches.append(list(batch))
        return {"loss": 0.0}


def _offline(cls, rows, tok, **cfg):
    t = object.__new__(cls)
    base = dict(epochs=1, batch_size=2, max_prompt_tokens=8, max_new_tokens=8, mini_bs=2,
                gradient_accumulation_steps=None, max_steps=None, save_path=None, save_interval=100,
                chat_template_enable_thinking=None)
    base.update(cfg)
    t.config = SimpleNamespace(**base)
    t.dataset, t.areno, t.loss_fn = rows, _Areno(tok), (lambda *a, **k: None)
    t.logger = logging.getLogger("test.offline")
    return t


def test_sft_batches_rows_and_reports_what_it_skipped(caplog):
    tok = FakeTokenizer()
    rows = [{"prompt": f"q {i}", "response": "an answer"} for i in range(3)] + [{"prompt": "q", "response": ""}]
    t = _offline(SFTTrainer, rows, tok)
    with caplog.at_level(logging.INFO):
        batches = list(t._iter_train_batches(tok))
    assert [len(b) for b in batches] == [2, 1] and "skipped_long_or_empty=1" in caplog.text


def test_sft_with_nothing_left_is_an_error():
    tok = FakeTokenizer()
    t = _offline(SFTTrainer, [{"prompt": "p", "response": ""}, {"prompt": "a b c d e f g h i j", "response": "r"}], tok)
    with pytest.raises(ValueError, match="no valid training rows.*scanned 2 row"):
        list(t._iter_train_batches(tok))


def test_offline_loop_trains_every_batch_and_stops_at_max_steps():
    tok = FakeTokenizer()
    rows = [{"prompt": f"q {i}", "response": "an answer"} for i in range(6)]
    t = _offline(SFTTrainer, rows, tok, epochs=2, max_steps=4)
    t._maybe_save = lambda epoch, step: None
    t._reached_max_steps = lambda epoch, step: step >= 4
    t._fit_initialized()
    assert [len(b) for b in t.areno.batches] == [2, 2, 2, 2]          # three per epoch, cut in the second epoch


# -------------------------------------------------------------------------------------------------- DPO rows

def test_dpo_rows_need_chosen_and_rejected_and_a_prompt_for_text():
    tok = FakeTokenizer()
    with pytest.raises(ValueError, match="`chosen` and `rejected`"):
        record_to_train_pair({"prompt": "p", "chosen": "c"}, tok, max_seq_len=32)
    with pytest.raises(ValueError, match="must contain `prompt`"):
        record_to_train_pair({"chosen": "c", "rejected": "r"}, tok, max_seq_len=32)


def test_dpo_text_pair_shares_the_prompt_and_keeps_chosen_first():
    tok = FakeTokenizer()
    pair = record_to_train_pair({"prompt": "which one", "chosen": "the good one", "rejected": "bad"}, tok, max_seq_len=32)
    chosen, rejected = pair
    n_p = len(tok.encode("which one"))
    assert chosen.tokens[:n_p] == rejected.tokens[:n_p] == tok.encode("which one")
    assert chosen.tokens[n_p:-1] == tok.encode("the good one") and rejected.tokens[n_p:-1] == tok.encode("bad")
    assert chosen.prompt_mask == [True] * n_p + [False] * 4 and rejected.prompt_mask == [True] * n_p + [False] * 2
    assert chosen.tokens[-1] == rejected.tokens[-1] == tok.eos_token_id


def test_dpo_message_pair_takes_the_common_prefix_as_prompt():
    tok = TemplateTokenizer()
    user = {"role": "user", "content": "pick"}
    pair = record_to_train_pair({"chosen": [user, {"role": "assistant", "content": "yes please"}],
                                 "rejected": [user, {"role": "assistant", "content": "no"}]}, tok, max_seq_len=32)
    chosen, rejected = pair
    shared = len(tok.encode("[user] pick [assistant]"))
    assert chosen.prompt_mask == [True] * shared + [False] * 2 and rejected.prompt_mask == [True] * shared + [False]
    assert tok.calls[0]["gen"] is False                       # whole conversations: no generation prompt


def test_dpo_message_prompt_with_text_answers():
    tok = TemplateTokenizer()
    pair = record_to_train_pair({"prompt": [{"role": "user", "content": "pick"}], "chosen": "a", "rejected": "b"}, tok,
                                max_seq_len=32)
    assert pair[0].tokens[:3] == tok.encode("[user] pick [assistant]") and tok.calls[0]["gen"] is True
    plain = FakeTokenizer()
    ids = encode_prompt_value(plain, [{"role": "user", "content": "pick"}])
    assert ids == plain.encode("user: pick")


def test_dpo_drops_pairs_that_are_too_long_or_have_no_answer_tokens():
    tok = FakeTokenizer()
    row = {"prompt": "p", "chosen": "a b c d e f", "rejected": "x"}
    assert record_to_train_pair(row, tok, max_seq_len=8) is not None
    assert record_to_train_pair(row, tok, max_seq_len=7) is None          # 1 + 6 + EOS = 8 tokens in the chosen row
    same = [{"role": "user", "content": "u"}]
    assert record_to_train_pair({"chosen": same, "rejected": same}, TemplateTokenizer(), max_seq_len=32) is None


def test_dpo_wants_an_even_mini_batch():
    with pytest.raises(ValueError, match="mini-bs to be even"):
        DPOTrainer(SimpleNamespace(mini_bs=3), instance=None, dataset=[], loss_fn=lambda **k: None)


def test_dpo_batches_hold_whole_pairs_and_count_pairs(caplog):
    tok = FakeTokenizer()
    rows = [{"prompt": f"p {i}", "chosen": "good", "rejected": "bad"} for i in range(3)]
    rows.insert(1, {"prompt": "p", "chosen": "a b c d e f g h i j k l m n o p q r", "rejected": "x"})
    t = _offline(DPOTrainer, rows, tok)
    with caplog.at_level(logging.INFO):
        batches = list(t._iter_train_batches(tok))
    assert [len(b) for b in batches] == [4, 2] and t._count(batches[0]) == 2
    assert "skipped_invalid_or_long=1" in caplog.text
    for b in batches:
        for chosen, rejected in zip(b[0::2], b[1::2]):
            assert chosen.tokens[-2] == tok.encode("good")[0] and rejected.tokens[-2] == tok.encode("bad")[0]


def test_dpo_fills_reference_logprobs_before_training():
    tok = FakeTokenizer()
    t = _offline(DPOTrainer, [], tok)
    pair = record_to_train_pair({"prompt": "p", "chosen": "c", "rejected": "r"}, tok, max_seq_len=32)
    t.areno.score_logprobs = lambda role, rows: [[-0.5] * len(r) for r in rows]
    extra = t._before_train(pair, 0, 0)
    assert pair[0].ref_logprobs == [-0.5] * len(pair[0].tokens) and pair[1].values == [0.0] * len(pair[1].tokens)
    assert extra["ref_logprob_forward_time_s"] >= 0.0
    t.areno.score_logprobs = lambda role, rows: [[0.0]] * len(rows)
    with pytest.raises(ValueError, match="misaligned"):
        t._before_train(pair, 0, 1)


# ----------------------------------------------------------------------------------------------- small helpers

def test_record_field_helpers_only_look_at_the_named_keys():
    rec = {"question": "q", "messages": [{"role": "user", "content": "m"}], "n": 3, "blank": None}
    assert first_value(rec, ("prompt", "question")) == "q" and first_value(rec, ("messages",)) == rec["messages"]
    assert first_value(rec, ("n", "blank", "absent")) is None
    assert has_any(rec, ("prompt", "question")) and not has_any(rec, ("n", "messages"))
    assert first_text(rec, ("prompt", "question")) == "q"
    with pytest.raises(KeyError):
        first_text(rec, ("prompt", "n"))


def test_conversations_without_a_template_become_role_lines():
    tok = FakeTokenizer()
    ids = apply_chat_template(tok, [{"role": "user", "content": "hi"}, {"content": "yo"}])
    assert ids == tok.encode("user: hi\nuser: yo")


def test_prompt_response_helper():
    tok = FakeTokenizer()
    toks, mask = prompt_response_to_tokens_and_mask("a b", "c", tok, eos_token_id=2)
    assert toks == tok.encode("a b") + tok.encode("c") + [2] and mask == [True, True, False, False]


# -------------------------------------------------------------------------------------------------- tokenizer API

def test_eos_ids_merge_tokenizer_config_and_text_config(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"eos_token_id": [7, 2], "text_config": {"eos_token_id": 9}}))
    tok = SimpleNamespace(eos_token_id=2)
    assert eos_token_ids(tmp_path, tok) == (2, 7, 9)
    assert eos_token_ids(tmp_path / "absent", tok) == (2,)
    assert eos_token_ids(tmp_path / "absent", SimpleNamespace(eos_token_id=None)) == ()
    (tmp_path / "config.json").write_text(json.dumps({"eos_token_id": True}))          # a bool is not an id
    assert eos_token_ids(tmp_path, SimpleNamespace(eos_token_id=[4, 4, "x"])) == (4,)


def test_generation_prompt_applies_the_template_once():
    tok = TemplateTokenizer()
    assert encode_generation_prompt(tok, "hello") == tok.encode("[user] hello [assistant]") and len(tok.calls) == 1
    pre = "<|im_start|>user hello"
    assert looks_chat_formatted(pre) and encode_generation_prompt(tok, pre) == tok.encode(pre) and len(tok.calls) == 1
    plain = FakeTokenizer()
    assert encode_generation_prompt(plain, "hello") == plain.encode("hello")


def test_thinking_switch_reaches_templates_that_take_it():
    tok = TemplateTokenizer()
    configure_chat_template_enable_thinking(tok, False)
    assert encode_generation_prompt(tok, "hello") == tok.encode("[user] hello [assistant] [nothink]")
    assert tok.calls[-1]["enable_thinking"] is False
    configure_chat_template_enable_thinking(tok, None)                    # back to the template's default
    encode_generation_prompt(tok, "hello")
    assert "enable_thinking" not in tok.calls[-1]
    configure_chat_template_enable_thinking(tok, None)                    # idempotent


def test_thinking_switch_is_dropped_for_templates_that_refuse_it():
    tok = TemplateTokenizer(accepts_thinking=False)
    configure_chat_template_enable_thinking(tok, True)
    assert encode_generation_prompt(tok, "hello") == tok.encode("[user] hello [assistant]")
    assert len(tok.calls) == 1 and "enable_thinking" not in tok.calls[0]

    class Broken(TemplateTokenizer):
        def apply_chat_template(self, *a, **kw):
            raise TypeError("unrelated")

    with pytest.raises(TypeError, match="unrelated"):
        apply_chat_template_with_options(Broken(), [{"role": "user", "content": "x"}], tokenize=True)


def test_token_ids_from_every_shape_a_tokenizer_returns():
    import numpy as np
    import torch

    assert normalize_token_ids([1, 2]) == [1, 2] and normalize_token_ids((3,)) == [3]
    assert normalize_token_ids(SimpleNamespace(ids=[4, 5])) == [4, 5]
    assert normalize_token_ids(SimpleNamespace(input_ids=[[6, 7]])) == [6, 7]
    assert normalize_token_ids([SimpleNamespace(ids=[8])]) == [8]
    assert normalize_token_ids(torch.tensor([[9, 10]])) == [9, 10] and normalize_token_ids(np.array([11])) == [11]
    assert normalize_token_ids([]) == []
    for bad in ([[1], [2]], [SimpleNamespace(ids=[1]), SimpleNamespace(ids=[2])], "text", 5, [object()]):
        with pytest.raises(TypeError):
            normalize_token_ids(bad)


# --------------------------------------------------------------------------------------------------- data models

def test_sampling_defaults_do_not_assume_a_backend():
    p = SamplingParams()
    assert (p.greedy, p.top_p, p.top_k, p.max_new_tokens, p.temperature) == (False, 1.0, -1, 16, 1.0)
    assert p.stop is None and p.stop_token_ids is None and p.max_context_len is None and p.max_prompt_len is None
    assert p.ignore_eos is False and p.skip_special_tokens is True and p.min_new_tokens == 0 and p.seed is None
    q = p.model_copy()
    q.max_new_tokens = 4
    assert p.max_new_tokens == 16


def test_train_sequences_do_not_share_their_default_lists():
    a, b = TrainSequence(), TrainSequence()
    a.tokens.append(1)
    a.ref_logprobs.append(0.5)
    assert b.tokens == [] and b.ref_logprobs == [] and (a.reward, a.eos_token_id) == (0.0, 0)
    r1, r2 = RolloutResult(), RolloutResult()
    r1.sequences.append(RolloutSequence(resp_tokens=[1], resp_logprobs=[-1.0]))
    assert r2.sequences == [] and RolloutSequence().resp_tokens == []


def test_backend_config_must_be_an_areno_config():
    from areno_b200.api import ArenoConfig, Trainer

    with pytest.raises(TypeError):
        Trainer(1, "ckpt", custom_config={"tp_size": 1}).init()
    cfg = ArenoConfig(tp_size=1)
    assert Trainer(1, "ckpt", custom_config=cfg) is not None
