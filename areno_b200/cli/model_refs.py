"""Model references: a local directory is used as is; anything else is treated as a Hugging Face
repo id and resolved with ``snapshot_download`` (``areno/cli/model_refs.py:11-44`` in the reference)."""

from __future__ import annotations

import os
from dataclasses import fields, is_dataclass, replace
from typing import Any

MODEL_REF_FIELDS = ("ckpt", "ref_ckpt", "reward_ckpt", "critic_ckpt", "model_path")


def resolve_model_path(ref: str | None) -> str | None:
    if ref is None:
        return None
    expanded = os.path.expanduser(str(ref))
    if os.path.isdir(expanded):
        return os.path.abspath(expanded)
    if os.path.sep in expanded and expanded.startswith((".", os.path.sep, "~")):
        raise FileNotFoundError(f"model path does not exist: {ref}")
    try:
        from huggingface_hub import snapshot_download
    except ImportError as exc:  # pragma: no cover
        raise FileNotFoundError(f"{ref!r} is not a local directory and huggingface_hub is not installed") from exc
    return snapshot_download(repo_id=str(ref))


def resolve_model_ref(model_ref: str, cache: dict[str, str] | None = None) -> str:
    """``resolve_model_path`` with a cache keyed by the reference: several roles that name the same repo id are
    resolved (and, the first time, downloaded) once (``areno/cli/model_refs.py:11-26``)."""
    if cache is not None and model_ref in cache:
        return cache[model_ref]
    resolved = resolve_model_path(model_ref)
    if cache is not None:
        cache[model_ref] = resolved
    return resolved


def resolve_model_refs_for_config(config: Any) -> Any:
    """Return a copy of a trainer config with every checkpoint reference resolved to a directory."""
    if not is_dataclass(config):
        return config
    names = {f.name for f in fields(config)}
    updates, cache = {}, {}
    for name in MODEL_REF_FIELDS:
        if name in names and getattr(config, name):
            updates[name] = resolve_model_ref(getattr(config, name), cache)
    return replace(config, **updates) if updates else config
