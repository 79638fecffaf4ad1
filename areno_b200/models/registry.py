"""Adapter registry: first match on the HF config wins; thread-safe registration
(``areno/models/registry.py:30-91`` in the reference)."""

from __future__ import annotations

import json
import os
import threading
from typing import Any

from .base import ModelAdapter

_lock = threading.RLock()
_adapters: list[ModelAdapter] = []
_bundled_loaded = False


def register_adapter(adapter: ModelAdapter | type[ModelAdapter]) -> ModelAdapter:
    inst = adapter() if isinstance(adapter, type) else adapter
    if not inst.name:
        raise ValueError("adapter must define a non-empty name")
    with _lock:
        for i, a in enumerate(_adapters):
            if a.name == inst.name:
                _adapters[i] = inst
                return inst
        _adapters.append(inst)
    return inst


def _ensure_bundled() -> None:
    global _bundled_loaded
    with _lock:
        if _bundled_loaded:
            return
        _bundled_loaded = True
        from . import register_models

        register_models()


def list_adapters() -> list[str]:
    _ensure_bundled()
    with _lock:
        return [a.name for a in _adapters]


def get_adapter(name: str) -> ModelAdapter:
    _ensure_bundled()
    with _lock:
        for a in _adapters:
            if a.name == name:
                return a
    raise KeyError(f"no model adapter named {name!r}; known: {list_adapters()}")


def find_adapter(hf_config: dict[str, Any]) -> ModelAdapter:
    _ensure_bundled()
    with _lock:
        for a in _adapters:
            if a.match_hf_config(hf_config):
                return a
    raise ValueError(
        f"no model adapter matches model_type={hf_config.get('model_type')!r} "
        f"architectures={hf_config.get('architectures')!r}; known adapters: {list_adapters()}")


def read_hf_config(model_path: str) -> dict[str, Any]:
    with open(os.path.join(model_path, "config.json")) as f:
        return json.load(f)


def config_from_pretrained(model_path: str):
    hf = read_hf_config(model_path)
    adapter = find_adapter(hf)
    return adapter, adapter.config_from_hf(hf)


# ---------------------------------------------------------------------------------------------------------------
# Dispatch helpers under the names of the reference's registry (``areno/models/registry.py:50-116``).

def load_model_plugins() -> None:
    """Register the bundled families (idempotent, thread-safe)."""
    _ensure_bundled()


def adapter_from_hf(model_path: str) -> ModelAdapter:
    return find_adapter(read_hf_config(str(model_path)))


def config_from_hf(model_path: str):
    return config_from_pretrained(str(model_path))[1]


def build_model(config, device="cpu"):
    return get_adapter(config.model_type).build(config, device=device)


def load_model_weights(model, config, model_path: str) -> None:
    get_adapter(config.model_type).load_weights(model, str(model_path), config)


def save_model_weights(model, config, output_path: str, source_path: str | None = None):
    """Save through the family's adapter.  Wrappers that keep the module under ``_orig_mod`` are peeled off first."""
    while getattr(model, "_orig_mod", None) is not None:
        model = model._orig_mod
    return get_adapter(config.model_type).save_weights(model, str(output_path), config, source_path)
