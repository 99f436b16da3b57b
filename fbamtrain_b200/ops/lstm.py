"""LSTM over a whole sequence on the GPU."""
from __future__ import annotations

from . import reference as ref


def lstm_sequence(x, w_ih, w_hh, b_ih, b_hh, h0, c0, compute_dtype):
    # Interim: per-step PyTorch ops.  The persistent recurrent kernel replaces this.
    return ref.lstm_sequence(x, w_ih, w_hh, b_ih, b_hh, h0, c0, compute_dtype)
