"""Levelled logger.

Lines look like ``YYYY-mm-dd HH:MM:SS - LEVEL: message`` on stdout; the threshold comes from the
``FBAMTRAIN_LOG_LEVEL`` environment variable and defaults to ``ERR``; ``FATAL`` and ``BUG`` end the
process (reference: ``src/logger.cpp:28-56, 66-95``).
"""
from __future__ import annotations

import os
import sys
import threading
import time

_LEVELS = {"DEBUG": 0, "INFO": 1, "WARN": 2, "ERR": 3, "FATAL": 4, "BUG": 5}
_lock = threading.Lock()


def _threshold() -> int:
    raw = os.environ.get("FBAMTRAIN_LOG_LEVEL", "ERR").upper()
    raw = {"ERROR": "ERR", "WARNING": "WARN"}.get(raw, raw)
    return _LEVELS.get(raw, _LEVELS["ERR"])


def enabled(level: str) -> bool:
    """Whether a message of this level would be printed."""
    return _LEVELS.get(level.upper(), _LEVELS["ERR"]) >= _threshold()


def LOG(level: str, message: str) -> None:
    level = level.upper()
    rank = _LEVELS.get(level, _LEVELS["ERR"])
    if rank >= _threshold():
        stamp = time.strftime("%Y-%m-%d %H:%M:%S")
        with _lock:
            sys.stdout.write(f"{stamp} - {level}: {message}\n")
            sys.stdout.flush()
    if level in ("FATAL", "BUG"):
        sys.exit(1)
