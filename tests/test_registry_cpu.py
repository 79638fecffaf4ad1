"""Model-adapter registry: bundled families, first-match dispatch on the HF config, replacement by name, concurrent
registration, error messages."""

from __future__ import annotations

import threading

import pytest

from areno_b200.models import registry
from areno_b200.models.base import ModelAdapter

BUNDLED = {"llama", "qwen2", "qwen3", "qwen3_moe", "qwen3_5", "qwen3_5_moe", "minicpmv46", "gemma4", "bailing_moe_linear_v2"}


def test_bundled_families_and_dispatch_on_hf_config():
    assert BUNDLED <= set(registry.list_adapters())
    cases = [({"model_type": "qwen2"}, "qwen2"), ({"model_type": "llama"}, "llama"), ({"model_type": "qwen3_moe"}, "qwen3_moe"),
             ({"model_type": "qwen3_5_moe"}, "qwen3_5_moe"), ({"model_type": "qwen3_5"}, "qwen3_5"),
             ({"architectures": ["Qwen3_5ForConditionalGeneration"]}, "qwen3_5"), ({"model_type": "minicpmv4_6"}, "minicpmv46"),
             ({"model_type": "gemma4", "text_config": {"model_type": "gemma4_text"}}, "gemma4"),
             ({"architectures": ["BailingMoeV2_5ForCausalLM"]}, "bailing_moe_linear_v2")]
    for hf, want in cases:
        assert registry.find_adapter(hf).name == want, hf
    with pytest.raises(ValueError, match="no model adapter matches"):
        registry.find_adapter({"model_type": "not-a-model"})
    with pytest.raises(KeyError, match="known"):
        registry.get_adapter("not-a-model")


class _Toy(ModelAdapter):
    name = "toy"
    tag = 0

    def match_hf_config(self, hf):
        return hf.get("model_type") == "toy"

    def config_from_hf(self, hf):
        return {"tag": self.tag}

    def build(self, config, device="cpu"):
        raise NotImplementedError

    def load_weights(self, model, path, config):
        raise NotImplementedError

    def save_weights(self, model, path, config, source_path=None):
        raise NotImplementedError


def test_registration_replaces_by_name_and_survives_threads(tmp_path):
    import json

    with pytest.raises(ValueError):
        registry.register_adapter(type("NoName", (_Toy,), {"name": ""}))
    first = registry.register_adapter(_Toy)
    assert registry.get_adapter("toy") is first
    second = registry.register_adapter(type("Toy2", (_Toy,), {"tag": 2}))
    assert registry.get_adapter("toy") is second and registry.list_adapters().count("toy") == 1     # replaced, not added
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "toy"}))
    adapter, cfg = registry.config_from_pretrained(str(tmp_path))
    assert adapter is second and cfg == {"tag": 2}

    errors = []

    def hammer(i):
        try:
            for j in range(50):
                registry.register_adapter(type(f"T{i}_{j}", (_Toy,), {"name": f"toy_{i}", "tag": j}))
                assert registry.get_adapter(f"toy_{i}").tag <= j
                registry.find_adapter({"model_type": "qwen2"})
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=hammer, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors
    names = registry.list_adapters()
    assert all(names.count(f"toy_{i}") == 1 for i in range(8)) and BUNDLED <= set(names)


def test_dispatch_helpers_build_load_and_save_through_the_family_adapter(tmp_path):
    import torch

    from areno_b200.parallel.context import single_process_context
    from tests.helpers import write_tiny_checkpoint

    single_process_context()
    src = str(tmp_path / "src")
    write_tiny_checkpoint(src, seed=4)
    registry.load_model_plugins()
    assert registry.adapter_from_hf(src).name == "qwen2"
    cfg = registry.config_from_hf(src)
    model = registry.build_model(cfg)
    registry.load_model_weights(model, cfg, src)

    class Wrapped:                                   # what a compiling wrapper looks like from outside
        def __init__(self, inner):
            self._orig_mod = inner

    out = str(tmp_path / "out")
    registry.save_model_weights(Wrapped(Wrapped(model)), cfg, out, src)
    again = registry.build_model(registry.config_from_hf(out))
    registry.load_model_weights(again, cfg, out)
    for (n, a), (_, b) in zip(model.named_parameters(), again.named_parameters()):
        assert torch.equal(a, b), n
