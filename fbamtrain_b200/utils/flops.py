"""FLOP accounting with a useful / total split.

Every tensor-core op adds its FLOPs here from the host when it is launched (2·M·N·K for a GEMM, the implicit-GEMM
count for a convolution, 4·B·H·T²·D for an attention forward, ...).  Work done under :func:`not_useful` —
recomputation of activations that a memory-unconstrained run would have kept — counts towards ``total`` only, so
``useful / time / peak`` is the model FLOP utilisation and ``total / time / peak`` the hardware utilisation
(reference: per-entry ``flop_estimate`` + ``is_useful`` in ``tensorlib/include/execution_plan.h:21-87``; recompute
GEMMs flagged not-useful in ``tensorlib/src/streaming_lstm_bwd.cpp:1229, 1236``).
"""
from __future__ import annotations

import threading
from contextlib import contextmanager
from typing import Tuple

from . import plan

_lock = threading.Lock()       # backward runs on autograd worker threads
_total = 0.0
_useful = 0.0
_local = threading.local()


def add(flops: float) -> None:
    global _total, _useful
    useful = not getattr(_local, "depth", 0)
    with _lock:
        _total += flops
        if useful:
            _useful += flops
    recording = plan.active()
    if recording is not None:
        recording.on_flops(flops, useful)


@contextmanager
def not_useful():
    """FLOPs added inside this block (on this thread) are recomputation."""
    _local.depth = getattr(_local, "depth", 0) + 1
    try:
        yield
    finally:
        _local.depth -= 1


def snapshot() -> Tuple[float, float]:
    """``(total, useful)`` FLOPs launched since the last :func:`reset`."""
    with _lock:
        return _total, _useful


def reset() -> None:
    global _total, _useful
    with _lock:
        _total = _useful = 0.0
