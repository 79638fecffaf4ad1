"""CPU end-to-end checks of the inference loop against a full (non-cached) forward."""

import pytest
import torch

from areno_b200.engine.config import ModelConfig
from areno_b200.engine.inference import InferenceEngine, SamplingParams
from areno_b200.models.dense import DenseCausalLM, TrainMeta, init_weights
from areno_b200.ops.attention import build_varlen_meta
from areno_b200.parallel.context import single_process_context


def tiny_config(**kw):
    base = dict(model_type="qwen2", vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, head_dim=32, rope_theta=1e4, qk_norm=False,
                qkv_bias=True, dtype=torch.float32)
    base.update(kw)
    return ModelConfig(**base)


def _full_logits(model, tokens):
    ids = torch.tensor(tokens)
    h = model(ids, torch.arange(len(tokens)), TrainMeta(build_varlen_meta([len(tokens)]), False)).hidden_states
    return model.compute_logits(h).float()


def _engine(model, **kw):
    single_process_context()
    args = dict(max_slots=4, max_model_len=256, max_prefill_tokens=64)
    args.update(kw)
    return InferenceEngine(model, 512, "cpu", **args)


def test_greedy_generation_matches_full_forward_with_continuous_batching_and_chunked_prefill():
    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 0)
    eng = _engine(model)
    g = torch.Generator().manual_seed(0)
    # 6 prompts through 4 slots (queueing), one prompt longer than the 64-token prefill budget (chunked)
    prompts = [torch.randint(3, 512, (n,), generator=g).tolist() for n in (20, 33, 100, 5, 12, 40)]
    out = eng.generate(prompts, SamplingParams(temperature=0.0), eos_token_ids=(), max_new_tokens=8)
    assert [len(t) for t in out.tokens] == [8] * 6
    assert out.finish_reasons == ["length"] * 6
    with torch.no_grad():
        for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
            logits = _full_logits(model, p + toks)
            pred = logits.argmax(-1)[len(p) - 1:-1].tolist()
            assert pred == toks
            ref = torch.log_softmax(logits, -1)[len(p) - 1:-1].gather(-1, torch.tensor(toks)[:, None]).squeeze(-1)
            assert torch.allclose(ref, torch.tensor(lps), atol=2e-2)


def test_stop_token_is_kept_and_min_new_tokens_masks_eos():
    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 1)
    eng = _engine(model)
    prompt = list(range(3, 20))
    base = eng.generate([prompt], SamplingParams(temperature=0.0), (), 6).tokens[0]
    eos = base[2]
    out = eng.generate([prompt], SamplingParams(temperature=0.0), (eos,), 6)
    assert out.tokens[0] == base[:3] and out.finish_reasons == ["stop"]
    out2 = eng.generate([prompt], SamplingParams(temperature=0.0, min_new_tokens=4), (eos,), 6)
    assert len(out2.tokens[0]) >= 4 and eos not in out2.tokens[0][:3]
    # user stop ids stop too, suppressed ids are never produced
    out3 = eng.generate([prompt], SamplingParams(temperature=0.0, stop_token_ids=(base[1],)), (), 6)
    assert out3.tokens[0] == base[:2] and out3.finish_reasons == ["stop"]
    out4 = eng.generate([prompt], SamplingParams(temperature=0.0, suppress_token_ids=(base[0],)), (), 3)
    assert base[0] not in out4.tokens[0]


def test_fp8_kv_cache_close_to_bf16():
    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 2)
    prompt = list(range(5, 60))
    a = _engine(model).generate([prompt], SamplingParams(temperature=0.0), (), 4)
    b = _engine(model, kv_fp8=True).generate([prompt], SamplingParams(temperature=0.0), (), 4)
    assert abs(a.logprobs[0][0] - b.logprobs[0][0]) < 0.05


def test_sampling_is_reproducible_per_seed_and_differs_across_rows():
    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 3)
    eng = _engine(model)
    prompts = [list(range(3, 30))] * 3
    a = eng.generate(prompts, SamplingParams(temperature=1.0, seed=11), (), 5)
    b = eng.generate(prompts, SamplingParams(temperature=1.0, seed=11), (), 5)
    assert all(len(t) == 5 for t in a.tokens) and all(len(t) == 5 for t in b.tokens)


def test_training_state_sidecar_resumes_optimizer_and_step(tmp_path, monkeypatch):
    """With ARENO_SAVE_OPTIMIZER=1 a checkpoint also carries the optimizer shards and step counters; a worker
    started from that checkpoint continues exactly where the first one would have."""
    import torch

    from areno_b200.api import loss_fns
    from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig
    from areno_b200.engine.worker import RankWorker
    from areno_b200.parallel.context import single_process_context

    from .helpers import tiny_config

    single_process_context()

    def pack(seed):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(3, 512, (2, 24), generator=g)
        pm = torch.ones((2, 24), dtype=torch.bool)
        pm[:, 10:] = False
        return dict(input_ids=ids, lengths=torch.tensor([24, 24]), prompt_mask=pm, logprobs=torch.zeros((2, 24)),
                    advantages=torch.where(pm, torch.zeros(()), torch.ones(())) * torch.tensor([[1.0], [-1.0]]))

    cfg = tiny_config()
    ec = EngineConfig(model=cfg, dummy_load=True, seed=3, optimizer=OptimizerConfig(lr=1e-2),
                      runtime=RuntimeConfig(max_model_len=64, activation_checkpointing=False))
    a = RankWorker(ec, "cpu")
    a.loss_fn = loss_fns.grpo_loss_fn
    a.train([pack(1)])
    monkeypatch.setenv("ARENO_SAVE_OPTIMIZER", "1")
    path = str(tmp_path / "ckpt")
    a.save_checkpoint(path)
    import json
    import os
    meta = json.load(open(os.path.join(path, "areno_state", "state.json")))
    assert meta["global_step"] == 1 and meta["optimizer_step"] == 1 and meta["world_size"] == 1
    ec2 = EngineConfig(model=cfg, model_path=path, seed=99, optimizer=OptimizerConfig(lr=1e-2),
                       runtime=RuntimeConfig(max_model_len=64, activation_checkpointing=False))
    b = RankWorker(ec2, "cpu")
    b.loss_fn = loss_fns.grpo_loss_fn
    assert b.training_manager().global_step == 1 and b.trainer.optimizer.step_count == 1
    for ba, bb in zip(a.trainer.optimizer.buckets, b.trainer.optimizer.buckets):
        assert torch.equal(ba.m, bb.m) and torch.equal(ba.v, bb.v)
    a.train([pack(2)])
    b.train([pack(2)])
    for pa, pb in zip(a.model.parameters(), b.model.parameters()):
        assert torch.allclose(pa, pb, atol=1e-6)
    # without the side-car the same checkpoint starts from fresh optimizer state
    import shutil
    shutil.rmtree(os.path.join(path, "areno_state"))
    c = RankWorker(ec2, "cpu")
    assert c.training_manager().global_step == 0


def test_sequence_evicted_for_lack_of_kv_pages_is_requeued_and_completes():
    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 3)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 512, (n,), generator=g).tolist() for n in (60, 61, 30)]
    roomy = _engine(model).generate(prompts, SamplingParams(temperature=0.0), (), 24)
    # 4 pages of 64 tokens: the two 60-token prompts fit one page each until their contexts cross 64 tokens together
    tight = _engine(model, num_pages=4)
    out = tight.generate(prompts, SamplingParams(temperature=0.0), (), 24)
    assert [len(t) for t in out.tokens] == [24, 24, 24]
    assert out.finish_reasons == ["length"] * 3
    assert out.tokens == roomy.tokens
    for a, b in zip(out.logprobs, roomy.logprobs):
        assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=2e-2)
    assert any(r.kept_tokens for r in tight._requests.values())     # an eviction really happened


def test_check_token_ids_guard_reports_out_of_range_samples(monkeypatch):
    from areno_b200.engine import inference

    inference._check_token_ids([0, 5, 511], 512, "ok")
    with pytest.raises(RuntimeError, match=r"out of vocab range \[0, 512\).*bad_max=600"):
        inference._check_token_ids([3, 600, -2], 512, "sampled tokens")
    # wired into collection: with the guard on, a vocabulary smaller than what the sampler can emit is caught
    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 0)
    eng = _engine(model)
    monkeypatch.setattr(inference, "_CHECK_TOKEN_IDS", True)
    eng.generate([[5, 6, 7]], SamplingParams(temperature=0.0), (), 4)      # in range: passes
    eng.vocab = 1
    with pytest.raises(RuntimeError, match="out of vocab range"):
        eng.generate([[5, 6, 7]], SamplingParams(temperature=0.0), (), 4)


def test_seeded_request_dealt_over_data_parallel_rows_draws_each_sample_from_its_own_stream():
    """Two engines stand for two data-parallel rows that share a seeded request of four samples of one prompt: with
    the samples' positions in the request as stream ids, the rows reproduce what one engine generates for all four,
    and no two samples coincide; numbering the streams per row would make the rows repeat each other."""
    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 3)
    prompt = list(range(3, 30))
    params = SamplingParams(temperature=1.0, seed=11)
    whole = _engine(model).generate([prompt] * 4, params, (), 6)
    row0 = _engine(model).generate([prompt] * 2, params, (), 6, stream_ids=[0, 2])
    row1 = _engine(model).generate([prompt] * 2, params, (), 6, stream_ids=[1, 3])
    assert [row0.tokens[0], row1.tokens[0], row0.tokens[1], row1.tokens[1]] == whole.tokens
    assert len({tuple(t) for t in whole.tokens}) == 4
    local = _engine(model).generate([prompt] * 2, params, (), 6)            # default numbering: 0, 1
    assert local.tokens == whole.tokens[:2]
    with pytest.raises(ValueError, match="one random stream per prompt"):
        _engine(model).generate([prompt] * 2, params, (), 6, stream_ids=[0])


def test_unseeded_engines_of_different_data_parallel_rows_draw_different_noise():
    """Rows share the engine seed and number their requests alike; the row's number keeps their samples apart, while a
    seeded request reproduces on whichever row serves it."""
    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 3)
    prompt = list(range(3, 30))
    free = SamplingParams(temperature=1.0)
    row0 = _engine(model, seed=5, stream_salt=0).generate([prompt] * 2, free, (), 8)
    row1 = _engine(model, seed=5, stream_salt=1).generate([prompt] * 2, free, (), 8)
    again = _engine(model, seed=5, stream_salt=0).generate([prompt] * 2, free, (), 8)
    assert row0.tokens == again.tokens and row0.tokens[0] != row1.tokens[0] and row0.tokens[1] != row1.tokens[1]
    seeded = SamplingParams(temperature=1.0, seed=9)
    assert _engine(model, seed=5, stream_salt=0).generate([prompt], seeded, (), 8).tokens == \
        _engine(model, seed=5, stream_salt=3).generate([prompt], seeded, (), 8).tokens


def test_progress_line_names_the_data_parallel_row(caplog):
    import logging

    single_process_context()
    model = DenseCausalLM(tiny_config())
    init_weights(model, 3)
    eng = _engine(model)
    with caplog.at_level(logging.INFO, logger="areno"):
        eng.generate([list(range(3, 20))] * 2, SamplingParams(temperature=0.0), (), 6, progress_interval_s=1e-9)
    lines = [r.getMessage() for r in caplog.records if "decode progress" in r.getMessage()]
    assert lines and all("row=0/1" in ln and "decode_tok_s=" in ln and "running=" in ln for ln in lines)
