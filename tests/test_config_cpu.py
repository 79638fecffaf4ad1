"""Configuration validation on the CPU: dtype names, tensor-parallel shape rules, the engine layout (devices, data
parallel size, rollout layout, expert parallelism, KV page size) and moving nested packs between devices.  The
behaviours follow the reference's ``tests/test_config_data_cpu.py``."""

from __future__ import annotations

from collections import namedtuple

import pytest
import torch

from areno_b200.api.trainer_config import TrainerConfig
from areno_b200.engine.config import EngineConfig, OptimizerConfig, RuntimeConfig, parse_dtype
from areno_b200.engine.training import to_device
from areno_b200.models.registry import get_adapter
from tests.helpers import tiny_config


# ---------------------------------------------------------------------------------------------- dtype names

@pytest.mark.parametrize("name,want", [
    ("bf16", torch.bfloat16), ("bfloat16", torch.bfloat16), ("torch.bfloat16", torch.bfloat16),
    ("fp16", torch.float16), ("half", torch.float16), ("float16", torch.float16),
    ("float", torch.float32), ("fp32", torch.float32), ("Float32", torch.float32), (" float32 ", torch.float32),
])
def test_parse_dtype_aliases(name, want):
    assert parse_dtype(name) is want


def test_parse_dtype_default_and_objects():
    assert parse_dtype(None) is torch.bfloat16
    assert parse_dtype("", torch.float32) is torch.float32
    assert parse_dtype(torch.float16) is torch.float16


@pytest.mark.parametrize("bad", ["int8", "float64", "fp8", torch.int32, torch.float64])
def test_parse_dtype_rejects_what_the_kernels_do_not_compute_in(bad):
    with pytest.raises(ValueError, match="unsupported model dtype"):
        parse_dtype(bad)


def _hf(**kw):
    base = dict(model_type="qwen2", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128)
    base.update(kw)
    return base


def test_adapter_reads_dtype_aliases_and_refuses_unknown_names():
    adapter = get_adapter("qwen2")
    assert adapter.config_from_hf(_hf(torch_dtype="float16")).dtype is torch.float16
    assert adapter.config_from_hf(_hf(dtype="bf16")).dtype is torch.bfloat16
    assert adapter.config_from_hf(_hf()).dtype is torch.bfloat16
    with pytest.raises(ValueError, match="unsupported model dtype"):
        adapter.config_from_hf(_hf(torch_dtype="int8"))


# ------------------------------------------------------------------------------------- tensor-parallel shapes

def test_validate_tp_even_split():
    cfg = tiny_config(num_attention_heads=8, num_key_value_heads=4, intermediate_size=256)
    for tp in (1, 2, 4):
        cfg.validate_tp(tp)
        assert cfg.kv_replication(tp) == 1


def test_validate_tp_rejects_nonpositive():
    with pytest.raises(ValueError, match="tp_size must be >= 1"):
        tiny_config().validate_tp(0)


def test_validate_tp_query_heads_must_divide():
    cfg = tiny_config(num_attention_heads=6, num_key_value_heads=2)
    with pytest.raises(ValueError, match="num_attention_heads"):
        cfg.validate_tp(4)


def test_validate_tp_kv_heads_divide_or_are_replicated():
    cfg = tiny_config(num_attention_heads=8, num_key_value_heads=2)
    cfg.validate_tp(4)
    assert cfg.kv_replication(4) == 2
    cfg.validate_tp(8)
    assert cfg.kv_replication(8) == 4
    with pytest.raises(ValueError, match="num_key_value_heads"):
        tiny_config(num_attention_heads=8, num_key_value_heads=3).validate_tp(2)


def test_validate_tp_intermediate_and_experts():
    with pytest.raises(ValueError, match="intermediate_size"):
        tiny_config(num_attention_heads=4, num_key_value_heads=4, intermediate_size=250).validate_tp(4)
    with pytest.raises(ValueError, match="num_experts"):
        tiny_config(num_attention_heads=4, num_key_value_heads=4, num_experts=6).validate_tp(4)
    tiny_config(num_attention_heads=4, num_key_value_heads=4, num_experts=8).validate_tp(4)


def test_validate_tp_padded_heads_only_for_inference_and_known_families():
    cfg = tiny_config(model_type="qwen2", num_attention_heads=28, num_key_value_heads=4, intermediate_size=512)
    with pytest.raises(ValueError, match="num_attention_heads"):
        cfg.validate_tp(8)
    cfg.validate_tp(8, inference_only=True)
    other = tiny_config(model_type="gemma4", num_attention_heads=28, num_key_value_heads=4, intermediate_size=512)
    with pytest.raises(ValueError, match="num_attention_heads"):
        other.validate_tp(8, inference_only=True)
    # the uneven deal needs tp to be a multiple of the KV heads
    with pytest.raises(ValueError):
        tiny_config(num_attention_heads=28, num_key_value_heads=4, intermediate_size=512).validate_tp(6, inference_only=True)


def test_rotary_dim_is_even_and_partial():
    assert tiny_config(head_dim=32).rotary_dim == 32
    assert tiny_config(head_dim=32, partial_rotary_factor=0.5).rotary_dim == 16
    assert tiny_config(head_dim=30, partial_rotary_factor=0.5).rotary_dim == 14


# -------------------------------------------------------------------------------------------- engine layout

def test_engine_config_infers_devices_and_dp():
    cfg = EngineConfig(model=tiny_config(), tp_size=2, dp_size=2)
    assert cfg.devices == [0, 1, 2, 3] and cfg.world_size == 4 and cfg.rollout_tp == 2 and cfg.rollout_dp == 2
    cfg = EngineConfig(model=tiny_config(), tp_size=2, devices=[4, 5, 6, 7])
    assert cfg.dp_size == 2 and cfg.world_size == 4
    cfg = EngineConfig(model=tiny_config())
    assert cfg.devices == [0] and cfg.dp_size == 1


def test_engine_config_rejects_layouts_that_do_not_fit_the_devices():
    with pytest.raises(ValueError, match="multiple of tp_size"):
        EngineConfig(model=tiny_config(), tp_size=2, devices=[0, 1, 2])
    with pytest.raises(ValueError, match="does not match"):
        EngineConfig(model=tiny_config(), tp_size=2, dp_size=3, devices=[0, 1, 2, 3])
    with pytest.raises(ValueError, match="multiple of tp_size"):
        EngineConfig(model=tiny_config(), tp_size=0, devices=[0])


def test_engine_config_checks_the_model_against_tp():
    with pytest.raises(ValueError, match="num_attention_heads"):
        EngineConfig(model=tiny_config(num_attention_heads=6, num_key_value_heads=2), tp_size=4)


def test_engine_config_accepts_dict_sections():
    cfg = EngineConfig(model=tiny_config(), optimizer={"lr": 3e-5, "adam_8bit": True},
                       runtime={"kv_dtype": "fp8", "kv_block_size": 32})
    assert isinstance(cfg.optimizer, OptimizerConfig) and cfg.optimizer.lr == 3e-5 and cfg.optimizer.adam_8bit
    assert isinstance(cfg.runtime, RuntimeConfig) and cfg.runtime.kv_dtype == "fp8"


def test_engine_config_kv_block_multiple_of_16():
    with pytest.raises(ValueError, match="kv_block_size"):
        EngineConfig(model=tiny_config(), runtime=RuntimeConfig(kv_block_size=24))


def test_runtime_config_validates_names():
    with pytest.raises(ValueError, match="attn_backend"):
        RuntimeConfig(attn_backend="paged")
    with pytest.raises(ValueError, match="kv_dtype"):
        RuntimeConfig(kv_dtype="int4")
    assert RuntimeConfig(attn_backend="native").attn_backend == "native"


def test_rollout_tp_needs_a_data_parallel_training_layout():
    model = tiny_config(num_attention_heads=8, num_key_value_heads=4)
    cfg = EngineConfig(model=model, tp_size=1, dp_size=4, rollout_tp_size=2)
    assert cfg.rollout_tp == 2 and cfg.rollout_dp == 2
    with pytest.raises(ValueError, match="requires tp_size == 1"):
        EngineConfig(model=model, tp_size=2, dp_size=2, rollout_tp_size=4)
    with pytest.raises(ValueError, match="rollout_tp_size"):
        EngineConfig(model=model, tp_size=1, dp_size=4, rollout_tp_size=3)
    # same width as training: nothing to check
    assert EngineConfig(model=model, tp_size=2, dp_size=1, rollout_tp_size=2).rollout_dp == 1


def test_rollout_tp_may_pad_query_heads():
    model = tiny_config(num_attention_heads=28, num_key_value_heads=4, intermediate_size=512)
    cfg = EngineConfig(model=model, tp_size=1, dp_size=8, rollout_tp_size=8)
    assert cfg.rollout_dp == 1


def test_expert_parallel_layout_rules():
    moe = tiny_config(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64)
    cfg = EngineConfig(model=moe, tp_size=1, dp_size=4, expert_parallel=True)
    assert cfg.expert_parallel and cfg.world_size == 4
    with pytest.raises(ValueError, match="tp_size must be 1"):
        EngineConfig(model=moe, tp_size=2, dp_size=2, expert_parallel=True)
    with pytest.raises(ValueError, match="tp_size must be 1"):
        EngineConfig(model=moe, tp_size=1, dp_size=4, rollout_tp_size=2, expert_parallel=True)
    with pytest.raises(ValueError, match="num_experts divisible"):
        EngineConfig(model=moe, tp_size=1, dp_size=3, expert_parallel=True)
    with pytest.raises(ValueError, match="num_experts divisible"):
        EngineConfig(model=tiny_config(), tp_size=1, dp_size=2, expert_parallel=True)


def test_trainer_config_checks_expert_parallel_and_backend_names():
    ok = TrainerConfig(algo="grpo", ckpt="x", dataset_path="y", tp_size=1, world_size=4, expert_parallel=True)
    assert ok.expert_parallel
    with pytest.raises(ValueError, match="tp_size must be 1"):
        TrainerConfig(algo="grpo", ckpt="x", dataset_path="y", tp_size=2, world_size=4, expert_parallel=True)
    with pytest.raises(ValueError, match="attn_backend"):
        TrainerConfig(algo="grpo", ckpt="x", dataset_path="y", attn_backend="xformers")


# -------------------------------------------------------------------------------------------- nested packs

def test_to_device_walks_nested_containers():
    Pair = namedtuple("Pair", "a b")
    pack = {"ids": torch.arange(4), "meta": {"lens": [torch.tensor([1, 2]), 3], "name": "x"},
            "pair": Pair(torch.ones(2), None), "tup": (torch.zeros(1), "s")}
    out = to_device(pack, torch.device("cpu"))
    assert out["ids"] is pack["ids"]                      # already there: no copy
    assert out["meta"]["lens"][1] == 3 and out["meta"]["name"] == "x"
    assert isinstance(out["pair"], Pair) and out["pair"].b is None and torch.equal(out["pair"].a, torch.ones(2))
    assert isinstance(out["tup"], tuple) and out["tup"][1] == "s"
    meta = to_device(pack, torch.device("meta"))
    assert meta["ids"].device.type == "meta" and meta["meta"]["lens"][0].device.type == "meta"
    assert meta["pair"].a.device.type == "meta" and meta["tup"][0].device.type == "meta"
    assert pack["ids"].device.type == "cpu"               # the input is not modified
