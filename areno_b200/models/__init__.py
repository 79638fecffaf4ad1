"""Model families.  ``register_models`` installs the bundled adapters (idempotent)."""

from __future__ import annotations


def register_models() -> None:
    from .registry import register_adapter
    from . import dense_adapters

    for cls in dense_adapters.ADAPTERS:
        register_adapter(cls)
    try:
        from . import moe_adapters

        for cls in moe_adapters.ADAPTERS:
            register_adapter(cls)
    except ImportError:
        pass
    try:
        from . import gemma4_adapter

        for cls in gemma4_adapter.ADAPTERS:
            register_adapter(cls)
    except ImportError:
        pass
    try:
        from . import bailing_adapter

        for cls in bailing_adapter.ADAPTERS:
            register_adapter(cls)
    except ImportError:
        pass
    try:
        from . import hybrid_adapters

        for cls in hybrid_adapters.ADAPTERS:
            register_adapter(cls)
    except ImportError:
        pass
