"""Debug switches that stand in for a sanitizer on shared GPUs.

* ``FBAMTRAIN_SYNC_EVERY_OP=1`` — synchronise the device after every custom-op launch so an
  asynchronous failure is attributed to the op that caused it (reference:
  ``tensorlib/src/execution_backend.cpp:39-43, 619-622``).
* ``FBAMTRAIN_POISON_ALLOC=1`` — fill every buffer obtained through :func:`fresh` with NaN (floats)
  or 0xFF bytes so reads of uninitialised memory surface in the numerics (the reference bisects the
  same class of bug by zero-filling op ranges, ``execution_backend.cpp:77-155``).
* ``FBAMTRAIN_DEBUG_KERNEL_LAUNCH=1`` — print one line per custom-kernel launch with its
  arguments (reference: ``execution_backend.cpp:796-803``).
* ``FBAMTRAIN_BREAK_ON_LAUNCH=<n | entry point name>`` — stop in the Python debugger (``breakpoint()``) right
  after the n-th native launch of the process, or after every launch of the named entry point, with the caller's
  frames on the stack (the reference breaks on a chosen tensor id, ``tensorlib/src/tensorlib.cpp:116-139``,
  ``tensorlib/src/cpudbg.cpp:7-21``).
"""
from __future__ import annotations

import os
import sys

import torch


def _flag(name: str) -> bool:
    return os.environ.get(name, "0") not in ("", "0", "false", "False")


PROFILE_LABELS = _flag("FBAMTRAIN_PROFILE_LABELS")   # wrap every native launch in a record_function range
SYNC_EVERY_OP = _flag("FBAMTRAIN_SYNC_EVERY_OP")
POISON_ALLOC = _flag("FBAMTRAIN_POISON_ALLOC")
DEBUG_KERNEL_LAUNCH = _flag("FBAMTRAIN_DEBUG_KERNEL_LAUNCH")
BREAK_ON_LAUNCH = os.environ.get("FBAMTRAIN_BREAK_ON_LAUNCH", "")


def break_requested(ordinal: int, entry_point: str) -> bool:
    """Whether the launch just made (the ``ordinal``-th of the process, 1-based) is the one to stop at."""
    if not BREAK_ON_LAUNCH:
        return False
    if BREAK_ON_LAUNCH.isdigit():
        return ordinal == int(BREAK_ON_LAUNCH)
    return entry_point == BREAK_ON_LAUNCH


def fresh(shape, dtype, device) -> torch.Tensor:
    """``torch.empty`` that honours the poison switch."""
    t = torch.empty(shape, dtype=dtype, device=device)
    if POISON_ALLOC and t.numel():
        if t.is_floating_point():
            t.fill_(float("nan"))
        else:
            t.view(torch.uint8).fill_(0xFF)
    return t


def label(name: str):
    """Profiler range around a native launch (only when FBAMTRAIN_PROFILE_LABELS is set)."""
    if PROFILE_LABELS:
        return torch.profiler.record_function(name)
    import contextlib
    return contextlib.nullcontext()


def after_launch(name: str, *args) -> None:
    if DEBUG_KERNEL_LAUNCH:
        desc = ", ".join(f"{tuple(a.shape)}:{str(a.dtype).replace('torch.', '')}" if isinstance(a, torch.Tensor)
                         else repr(a) for a in args)
        sys.stdout.write(f"[launch] {name}({desc})\n")
    if SYNC_EVERY_OP and torch.cuda.is_available():
        torch.cuda.synchronize()
