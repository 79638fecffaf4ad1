"""SDK end-to-end on CPU: Trainer -> native backend -> in-process worker (tiny model)."""

import asyncio
import os

import pytest

from areno_b200.api import ArenoConfig, SamplingParams, Trainer, TrainSequence, grpo_loss_fn, sft_loss_fn
from areno_b200.api.rewards import compute_group_advantages
from tests.helpers import FakeTokenizer, write_tiny_checkpoint


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("model") / "tiny")
    write_tiny_checkpoint(path, seed=0)
    return path


def _trainer(ckpt):
    cfg = ArenoConfig(tp_size=1, max_running_prompts=8, decode_progress_interval_s=0.0, launcher="inprocess",
                      optimizer={"lr": 1e-3, "grad_clip_norm": 1.0}, runtime={"max_model_len": 128})
    t = Trainer(1, ckpt, custom_config=cfg)
    t.init(tokenizer=FakeTokenizer(), eos_ids=(2,))
    return t


def test_rollout_train_save_cycle(ckpt, tmp_path):
    t = _trainer(ckpt)
    try:
        assert t.dp_size() == 1 and t.model_context_len() == 512
        prompts = [[5, 6, 7, 8], [9, 10, 11], [20, 21, 22, 23, 24]]
        with pytest.raises(RuntimeError):
            t.rollout_token_batch(prompts, 2, SamplingParams(max_new_tokens=4))
        params = SamplingParams(max_new_tokens=6, temperature=1.0, ignore_eos=True)
        with t.rollout_session(sampling_params=params):
            results = t.rollout_token_batch(prompts, 2, params)
        assert len(results) == 3 and all(len(r.sequences) == 2 for r in results)
        assert all(len(s.resp_tokens) == 6 and len(s.resp_logprobs) == 6 for r in results for s in r.sequences)
        batch = []
        for p, res in zip(prompts, results):
            rewards = [float(sum(s.resp_tokens) % 2) for s in res.sequences]
            for s, adv, rew in zip(res.sequences, compute_group_advantages(rewards), rewards):
                batch.append(TrainSequence(prompt_mask=[True] * len(p) + [False] * 6, tokens=p + s.resp_tokens,
                                           logprobs=[0.0] * len(p) + s.resp_logprobs,
                                           advantages=[0.0] * len(p) + [adv] * 6, reward=rew, eos_token_id=2))
        stats = t.train(batch, grpo_loss_fn, mini_bs=4)
        assert stats["global_step"] == 1 and stats["num_microbatches"] == 2
        # rollout and training kernels agree on the log-probs of the sampled tokens
        assert stats["logp_abs_diff_mean"] < 1e-3
        assert "step_rollout_time_s" in stats and "step_train_time_s" in stats and "grad_norm" in stats
        assert t.global_step == 0
        out = t.save_checkpoint(str(tmp_path / "saved"))
        assert os.path.exists(os.path.join(out, "model.safetensors.index.json"))
        assert os.path.exists(os.path.join(out, "config.json"))
    finally:
        t.close()


def test_async_rollouts_join_one_running_batch_and_sft_train(ckpt):
    t = _trainer(ckpt)
    try:
        params = SamplingParams(max_new_tokens=5, greedy=True, ignore_eos=True)

        async def run():
            async with t.rollout_session(sampling_params=params, proxy=False):
                return await asyncio.gather(*[t.rollout_token_batch_async([[7, 8, 9 + i]], 1, params) for i in range(5)])

        outs = asyncio.run(run())
        assert len(outs) == 5 and all(len(o[0].sequences[0].resp_tokens) == 5 for o in outs)
        # greedy: the same prompt gives the same completion whether batched alone or with others
        with t.rollout_session(sampling_params=params):
            alone = t.rollout_token_batch([[7, 8, 9]], 1, params)
        assert alone[0].sequences[0].resp_tokens == outs[0][0].sequences[0].resp_tokens
        seqs = [TrainSequence(prompt_mask=[True, True, False, False, False], tokens=[5, 6, 7, 8, 2],
                              logprobs=[0.0] * 5, advantages=[0.0] * 5, eos_token_id=2) for _ in range(4)]
        s1 = t.train(seqs, sft_loss_fn, mini_bs=2)
        s2 = t.train(seqs, sft_loss_fn, mini_bs=2)
        assert s2["sft_loss"] < s1["sft_loss"]
    finally:
        t.close()
