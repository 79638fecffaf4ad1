import json
import os

import torch

from areno_b200.engine.checkpoint import SafetensorsIndex, load_dense_checkpoint, owner_rank
from areno_b200.models.dense import DenseCausalLM, init_weights
from areno_b200.models.registry import config_from_pretrained
from areno_b200.parallel.context import single_process_context
from tests.helpers import tiny_config, write_tiny_checkpoint


def test_save_load_round_trip_and_hf_layout(tmp_path):
    path = str(tmp_path / "ckpt")
    cfg = write_tiny_checkpoint(path, seed=3)
    index = json.load(open(os.path.join(path, "model.safetensors.index.json")))
    assert index["metadata"]["areno_checkpoint_writer"] == "distributed_tp"
    assert os.path.exists(os.path.join(path, "model-00001-of-00001.safetensors"))
    keys = set(index["weight_map"])
    assert {"model.embed_tokens.weight", "model.norm.weight", "lm_head.weight",
            "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.bias",
            "model.layers.1.mlp.gate_proj.weight", "model.layers.1.mlp.down_proj.weight"} <= keys
    idx = SafetensorsIndex(path)
    assert idx.shape("model.layers.0.self_attn.q_proj.weight") == [128, 128]
    assert idx.shape("model.layers.0.self_attn.k_proj.weight") == [64, 128]
    assert idx.shape("model.layers.0.mlp.gate_proj.weight") == [256, 128]
    single_process_context()
    adapter, cfg2 = config_from_pretrained(path)
    assert adapter.name == "qwen2" and cfg2.hidden_size == cfg.hidden_size and cfg2.qkv_bias
    ref = DenseCausalLM(tiny_config())
    init_weights(ref, 3)
    model = DenseCausalLM(tiny_config())
    init_weights(model, 99)
    load_dense_checkpoint(model, path, cfg)
    for (n, a), (_, b) in zip(ref.named_parameters(), model.named_parameters()):
        assert torch.equal(a, b), n


def test_owner_rank_is_stable():
    assert owner_rank("model.norm.weight", 4) == owner_rank("model.norm.weight", 4)
    assert 0 <= owner_rank("x", 3) < 3
