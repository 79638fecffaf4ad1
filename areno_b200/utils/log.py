"""Package logger: ``areno`` namespace, level from ``ARENO_LOG_LEVEL`` (default INFO), one stream
handler, ``key=value`` message style.  Same environment contract as ``areno/engine/log.py:13-35``."""

from __future__ import annotations

import logging
import os

_LOGGER_NAME = "areno"
_configured = False


def get_logger(name: str | None = None) -> logging.Logger:
    global _configured
    root = logging.getLogger(_LOGGER_NAME)
    if not _configured:
        level = os.environ.get("ARENO_LOG_LEVEL", "INFO").upper()
        root.setLevel(getattr(logging, level, logging.INFO))
        if not root.handlers:
            handler = logging.StreamHandler()
            handler.setFormatter(logging.Formatter("[%(asctime)s] [%(levelname)s] [%(name)s] %(message)s"))
            root.addHandler(handler)
        root.propagate = False
        _configured = True
    return root if not name else root.getChild(name)
