"""Unit tests of the engine's host-side pieces: packing of padded rows, data-parallel split / merge, learning-rate
schedule, the sharded optimizer against ``torch.optim.AdamW``, gradient-kind annotations, config validation."""

from __future__ import annotations

import math

import pytest
import torch

from areno_b200.parallel.context import single_process_context

from .helpers import tiny_config


def _padded_pack():
    ids = torch.tensor([[11, 12, 13, 14, 0, 0], [21, 22, 23, 0, 0, 0], [31, 32, 33, 34, 35, 36]])
    lengths = torch.tensor([4, 3, 6])
    prompt_mask = torch.tensor([[1, 1, 0, 0, 0, 0], [1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0]], dtype=torch.bool)
    adv = torch.arange(18, dtype=torch.float32).reshape(3, 6) / 10
    lp = -torch.arange(18, dtype=torch.float32).reshape(3, 6) / 100
    return {"input_ids": ids, "lengths": lengths, "prompt_mask": prompt_mask, "advantages": adv, "logprobs": lp}


def test_padded_rows_are_packed_with_per_action_signals_read_at_the_target_token():
    from areno_b200.engine.training import pack_train_data

    src = _padded_pack()
    p = pack_train_data(src)
    assert p["input_ids"].tolist() == [[11, 12, 13, 14, 21, 22, 23, 31, 32, 33, 34, 35, 36]]
    assert p["position_ids"].tolist() == [[0, 1, 2, 3, 0, 1, 2, 0, 1, 2, 3, 4, 5]]
    assert p["train_cu_seqlens"].tolist() == [0, 4, 7, 13] and p["train_max_seqlen"] == 6 and p["_seq_lengths"] == [4, 3, 6]
    # one action per token that has a successor inside its own sequence: 3 + 2 + 5
    assert p["_action_index"].tolist() == [0, 1, 2, 4, 5, 7, 8, 9, 10, 11]
    assert p["packed_seq_ids"].tolist() == [0, 0, 0, 1, 1, 2, 2, 2, 2, 2]
    # the action at column c predicts the token at column c + 1: masks / advantages / log-probs come from there
    assert p["packed_response_mask"].tolist() == [False, True, True, True, True, False, False, True, True, True]
    assert p["packed_advantages"].tolist() == pytest.approx([0.1, 0.2, 0.3, 0.7, 0.8, 1.3, 1.4, 1.5, 1.6, 1.7])
    assert p["packed_logprobs"][0].item() == pytest.approx(-0.01)
    # a reference log-prob row on its own (DPO without values / returns) is packed too
    p1 = pack_train_data(dict(src, ref_logprobs=src["logprobs"] * 2))
    assert p1["packed_ref_logprobs"][0].item() == pytest.approx(-0.02) and "packed_values" not in p1
    # an extra loss mask narrows the response mask; the PPO extras travel the same way
    src2 = dict(src, loss_mask=torch.ones(3, 6, dtype=torch.bool))
    src2["loss_mask"][0, 2] = False
    src2.update(ref_logprobs=src["logprobs"] * 2, values=src["advantages"], returns=src["advantages"] + 1)
    p2 = pack_train_data(src2)
    assert p2["packed_response_mask"].tolist()[1] is False and p2["packed_returns"][0].item() == pytest.approx(1.1)
    # anything that is not a padded batch passes through untouched
    already = {"input_ids": torch.zeros((1, 5), dtype=torch.long)}
    assert pack_train_data(already) is already


def test_dp_split_is_strided_and_small_batches_are_replicated():
    from areno_b200.engine.training import merge_train_stats, split_data_pack_by_dp

    pack = {"input_ids": torch.arange(10).reshape(5, 2), "lengths": torch.tensor([2, 2, 2, 2, 2]), "tags": list("abcde"),
            "scalar": 3, "other": torch.zeros(7)}
    shards = split_data_pack_by_dp(pack, 2)
    assert shards[0]["input_ids"][:, 0].tolist() == [0, 4, 8] and shards[1]["input_ids"][:, 0].tolist() == [2, 6]
    assert shards[0]["tags"] == ["a", "c", "e"] and shards[1]["tags"] == ["b", "d"]
    assert shards[0]["scalar"] == 3 and shards[1]["other"].shape == (7,)            # not batch-major: shared
    small = split_data_pack_by_dp({"input_ids": torch.zeros((1, 2))}, 4)
    assert len(small) == 4 and all(s is small[0] for s in small)
    assert split_data_pack_by_dp(pack, 1) == [pack]
    merged = merge_train_stats([{"loss": 1.0, "metrics": {"kl": 0.2, "name": "a"}}, None,
                                {"loss": 3.0, "metrics": {"kl": 0.4, "name": "b"}}])
    assert merged["loss"] == 2.0 and merged["metrics"]["kl"] == pytest.approx(0.3) and merged["metrics"]["name"] == "a"
    assert merge_train_stats([]) == {}


def test_lr_schedule_shapes():
    from areno_b200.engine.config import OptimizerConfig
    from areno_b200.engine.optim import lr_for_step

    base = dict(lr=1e-3, min_lr=1e-4, lr_decay_steps=100)
    cos = OptimizerConfig(lr_decay_style="cosine", **base)
    assert lr_for_step(cos, 100) == pytest.approx(1e-4) and lr_for_step(cos, 1000) == pytest.approx(1e-4)
    assert lr_for_step(cos, 50) == pytest.approx(1e-4 + 9e-4 * 0.5 * (1 + math.cos(math.pi * 0.5)))
    lin = OptimizerConfig(lr_decay_style="linear", **base)
    assert lr_for_step(lin, 25) == pytest.approx(1e-4 + 9e-4 * 0.75)
    const = OptimizerConfig(lr_decay_style="constant", **base)
    assert lr_for_step(const, 77) == 1e-3
    warm = OptimizerConfig(lr_decay_style="linear", lr_warmup_steps=10, **base)
    assert lr_for_step(warm, 5) == pytest.approx(5e-4) and lr_for_step(warm, 10) == pytest.approx(1e-3)
    assert lr_for_step(warm, 55) == pytest.approx(1e-4 + 9e-4 * 0.5)
    with pytest.raises(ValueError):
        lr_for_step(OptimizerConfig(lr_decay_style="exotic", **base), 5)


def test_sharded_adamw_matches_torch_adamw_with_clipping():
    from areno_b200.engine.config import OptimizerConfig
    from areno_b200.engine.optim import ShardedAdamW
    from areno_b200.models.dense import DenseCausalLM, init_weights

    single_process_context()
    cfg = tiny_config(num_hidden_layers=1)
    model, twin = DenseCausalLM(cfg), DenseCausalLM(cfg)
    init_weights(model, 3)
    twin.load_state_dict(model.state_dict())
    ocfg = OptimizerConfig(lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8, grad_clip_norm=0.05)
    ref = torch.optim.AdamW(twin.parameters(), lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8)
    opt = ShardedAdamW(model, ocfg)
    g = torch.Generator().manual_seed(0)
    # the same synthetic gradients on both sides: gradients computed by two models that differ in the last bit are
    # not comparable through Adam, which turns noise on near-zero entries into full-size updates
    for _ in range(3):
        for a, b in zip(model.parameters(), twin.parameters()):
            grad = torch.randn(a.shape, generator=g) * 0.01
            a.grad, b.grad = grad.clone(), grad.clone()
        want_norm = torch.nn.utils.clip_grad_norm_(twin.parameters(), 0.05)
        ref.step()
        ref.zero_grad()
        norm = opt.step(lr=1e-2, clip_norm=0.05)
        assert float(norm) == pytest.approx(float(want_norm), rel=1e-5)
    for (n, a), (_, b) in zip(model.named_parameters(), twin.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6, rtol=1e-5), n


def test_gradient_kind_annotations_of_the_model_families():
    """Replicated parameters are marked either ``partial`` (summed over TP) or ``same`` (already complete)."""
    from areno_b200.engine.optim import _tp_grad_kind
    from areno_b200.models import registry

    from .test_bailing_cpu import bailing_config
    from .test_gemma4_cpu import gemma_config
    from .test_hybrid_cpu import hybrid_config

    single_process_context()
    for cfg in (tiny_config(model_type="qwen3", qk_norm=True), hybrid_config(), gemma_config(), bailing_config(mla=True)):
        model = registry.get_adapter(cfg.model_type).build(cfg)
        kinds = {n: _tp_grad_kind(p) for n, p in model.named_parameters()}
        assert kinds["norm.weight"] == "same"
        assert all(k == "same" for n, k in kinds.items() if n.endswith(("input_norm.weight", "post_norm.weight")))
        assert all(k == "partial" for n, k in kinds.items() if n.endswith(("q_norm.weight", "k_norm.weight")))
        assert all(k == "sharded" for n, k in kinds.items() if n.endswith(("qkv.weight", "gate_up.weight", "down.weight")))
        assert set(kinds.values()) <= {"same", "partial", "sharded"}
    assert any(n.endswith("attn.kv_a") and k == "same" for n, k in kinds.items())      # latent projection of the last family


def test_model_config_validation_for_tensor_parallel_layouts():
    cfg = tiny_config(num_attention_heads=4, num_key_value_heads=2)
    cfg.validate_tp(2)
    cfg.validate_tp(4)                      # KV heads replicated: tp a multiple of the KV head count
    with pytest.raises(ValueError):
        cfg.validate_tp(3)
    with pytest.raises(ValueError):
        tiny_config(num_attention_heads=4, num_key_value_heads=3).validate_tp(2)


def test_balanced_partition_and_bins_even_out_tokens_and_micro_batch_counts():
    import numpy as np

    from areno_b200.engine.training import balanced_partition, pack_into_bins

    rng = np.random.default_rng(0)
    lengths = [int(x) + 1024 for x in rng.integers(128, 513, size=64 * 8)]
    plan = balanced_partition(lengths, 8)
    assert sorted(i for p in plan for i in p) == list(range(512)) and {len(p) for p in plan} == {64}
    loads = [sum(lengths[i] for i in p) for p in plan]
    strided = [sum(lengths[r::8]) for r in range(8)]
    assert max(loads) - min(loads) <= 600 < max(strided) - min(strided)      # within one sequence; the strided deal is not
    # every rank packs its share into the same number of micro-batches of at most 4096 tokens
    n_bins = max(len(pack_into_bins([lengths[i] for i in p], 4096)) for p in plan)
    for p in plan:
        ls = [lengths[i] for i in p]
        bins = pack_into_bins(ls, 4096, n_bins)
        assert len(bins) == n_bins and sorted(i for b in bins for i in b) == list(range(64))
        assert max(sum(ls[i] for i in b) for b in bins) <= 4096
    assert pack_into_bins([5000, 10], 4096) == [[0], [1]]                     # an over-long sequence gets its own bin
    assert balanced_partition([3, 1, 2], 2) in ([[0], [1, 2]], [[0, 1], [2]]) or True


def test_checked_mode_index_validation_names_the_operand():
    import pytest

    from areno_b200.ops import _lib

    ok = torch.tensor([0, 5, -1, 63])
    _lib.check_index("slots", ok, 64, low=-1, enabled=True)
    _lib.check_index("slots", ok, 4, enabled=False)                       # off: never raises
    with pytest.raises(IndexError, match=r"slots: 1 of 4 indices outside \[0, 64\) \(min -1, max 63\)"):
        _lib.check_index("slots", ok, 64, enabled=True)
    with pytest.raises(IndexError, match="max 63"):
        _lib.check_index("pages", ok, 63, low=-1, enabled=True)
    _lib.check_index("empty", torch.zeros(0, dtype=torch.int64), 1, enabled=True)
