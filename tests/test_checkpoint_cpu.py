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
    assert os.path.exists(os.path.join(path, "model.safetensors"))
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


def test_index_reads_sharded_checkpoints_lazily_and_slices_without_loading_whole_tensors(tmp_path):
    import pytest
    from safetensors.torch import save_file

    d = tmp_path / "sharded"
    d.mkdir()
    a = torch.arange(24, dtype=torch.float32).reshape(6, 4)
    b = torch.arange(8, dtype=torch.float32).reshape(2, 4) + 100
    save_file({"a.weight": a}, str(d / "model-00001-of-00002.safetensors"))
    save_file({"b.weight": b}, str(d / "model-00002-of-00002.safetensors"))
    # without an index file the shards are discovered by listing the directory
    idx = SafetensorsIndex(str(d))
    assert sorted(idx.keys()) == ["a.weight", "b.weight"] and "a.weight" in idx and "c" not in idx
    assert idx.shape("a.weight") == [6, 4]
    assert torch.equal(idx.get_rows("a.weight", 2, 4), a[2:4]) and torch.equal(idx.get_cols("a.weight", 1, 3), a[:, 1:3])
    assert torch.equal(idx.get("b.weight"), b)
    idx.drop()                                               # closes the cached handles; reading reopens them
    assert torch.equal(idx.get("b.weight"), b)
    # with an index file only the listed names exist
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a.weight": "model-00001-of-00002.safetensors"}}))
    assert sorted(SafetensorsIndex(str(d)).keys()) == ["a.weight"]
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError):
        SafetensorsIndex(str(empty))


def test_missing_and_mismatched_tensors_are_reported(tmp_path):
    import pytest
    from safetensors.torch import load_file, save_file

    path = str(tmp_path / "ckpt")
    cfg = write_tiny_checkpoint(path, seed=1)
    fname = os.path.join(path, "model.safetensors")
    tensors = {k: v.clone() for k, v in load_file(fname).items()}     # private copies: the file is rewritten below
    single_process_context()
    # a required tensor is gone
    broken = dict(tensors)
    broken.pop("model.layers.0.self_attn.o_proj.weight")
    save_file(broken, fname, metadata={"format": "pt"})
    index = json.load(open(os.path.join(path, "model.safetensors.index.json")))
    index["weight_map"].pop("model.layers.0.self_attn.o_proj.weight")
    json.dump(index, open(os.path.join(path, "model.safetensors.index.json"), "w"))
    with pytest.raises(KeyError, match="o_proj"):
        load_dense_checkpoint(DenseCausalLM(tiny_config()), path, cfg)
    # a tensor of the wrong shape
    wrong = dict(tensors)
    wrong["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(7, 7)
    save_file(wrong, fname, metadata={"format": "pt"})
    index["weight_map"]["model.layers.0.self_attn.o_proj.weight"] = "model.safetensors"
    json.dump(index, open(os.path.join(path, "model.safetensors.index.json"), "w"))
    with pytest.raises(ValueError, match="shape mismatch"):
        load_dense_checkpoint(DenseCausalLM(tiny_config()), path, cfg)


def test_saving_from_a_source_directory_keeps_foreign_tensors_and_assets(tmp_path):
    from safetensors.torch import save_file

    from areno_b200.engine.checkpoint import save_dense_checkpoint

    src = str(tmp_path / "src")
    cfg = write_tiny_checkpoint(src, seed=2)
    # a tensor the text model does not own (a vision tower, say) and a tokenizer file next to the weights
    save_file({"vision.patch_embed.weight": torch.ones(3, 5)}, os.path.join(src, "model-vision.safetensors"))
    index = json.load(open(os.path.join(src, "model.safetensors.index.json")))
    index["weight_map"]["vision.patch_embed.weight"] = "model-vision.safetensors"
    json.dump(index, open(os.path.join(src, "model.safetensors.index.json"), "w"))
    open(os.path.join(src, "tokenizer_config.json"), "w").write('{"model_max_length": 99}')
    single_process_context()
    model = DenseCausalLM(tiny_config())
    load_dense_checkpoint(model, src, cfg)
    out = str(tmp_path / "out")
    save_dense_checkpoint(model, out, cfg, source_path=src)
    idx = SafetensorsIndex(out)
    assert torch.equal(idx.get("vision.patch_embed.weight"), torch.ones(3, 5))
    assert idx.weight_map["vision.patch_embed.weight"] == "model-passthrough.safetensors"
    assert json.load(open(os.path.join(out, "tokenizer_config.json")))["model_max_length"] == 99
    assert os.path.exists(os.path.join(out, "config.json"))
