"""Model families.  ``register_models`` installs the bundled adapters (idempotent: registration replaces by name)."""

from __future__ import annotations


def register_models() -> None:
    from . import bailing_adapter, dense_adapters, gemma4_adapter, hybrid_adapters, moe_adapters
    from .registry import register_adapter

    # first match wins when an HF config is looked up: plain dense families come first, the families that recognise
    # themselves by architecture names after them
    for module in (dense_adapters, moe_adapters, gemma4_adapter, bailing_adapter, hybrid_adapters):
        for cls in module.ADAPTERS:
            register_adapter(cls)
