"""Scoped NVTX ranges around training phases.

Phase names follow the reference's ``GPUTX_RANGE`` labels — ``fbamtrain::zero_grad``,
``fbamtrain::forward``, ``fbamtrain::frame_head_fwd``, ``fbamtrain::action_model_fwd_bwd``,
``fbamtrain::backward``, ``fbamtrain::frame_head_grad_allreduce``, ``fbamtrain::action_model_optim_step`` …
(reference: ``tensorlib/include/gputx.h:24-52``, ``src/main.cpp:3037-3733``).  Ranges are no-ops on
CPU or when ``FBAMTRAIN_NVTX=0``.
"""
from __future__ import annotations

import contextlib
import os

import torch

from . import plan

_ENABLED = os.environ.get("FBAMTRAIN_NVTX", "1") != "0"


@contextlib.contextmanager
def gputx_range(name: str):
    active = _ENABLED and torch.cuda.is_available()
    if active:
        torch.cuda.nvtx.range_push(name)
    recording = plan.active() is not None
    if recording:
        plan.push_phase(name)
    try:
        yield
    finally:
        if recording:
            plan.pop_phase()
        if active:
            torch.cuda.nvtx.range_pop()
