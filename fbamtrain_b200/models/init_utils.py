"""Seeded parameter initialisation.

Scheme of the reference: embeddings N(0, 1); Linear / conv / LSTM weights and biases
U(-1/sqrt(fan_in), +1/sqrt(fan_in)) (the LSTM's fan is its hidden size); RMSNorm gains 1;
``h0 = c0 = 0``; every tensor draws from its own seed, and seeds increase by one per tensor starting
at ``model_init_seed`` (reference: ``src/framehead_model.cpp:528-598``,
``tensorlib/include/linear.h:39-44``, ``tensorlib/include/streaming_lstm.h:68-74``).  The random
streams are PyTorch's CPU generator, so values differ from the reference's Philox fills while the
distributions match.
"""
from __future__ import annotations

import math

import torch


class SeedSequence:
    def __init__(self, seed: int):
        self.next_seed = int(seed)

    def take(self) -> int:
        s = self.next_seed
        self.next_seed += 1
        return s


def fill_normal_(t: torch.Tensor, seeds: SeedSequence) -> None:
    g = torch.Generator(device="cpu").manual_seed(seeds.take())
    with torch.no_grad():
        t.copy_(torch.randn(t.shape, generator=g, dtype=torch.float32).to(t.dtype))


def fill_uniform_fan_(t: torch.Tensor, fan_in: int, seeds: SeedSequence) -> None:
    g = torch.Generator(device="cpu").manual_seed(seeds.take())
    bound = 1.0 / math.sqrt(max(1, fan_in))
    with torch.no_grad():
        t.copy_(((torch.rand(t.shape, generator=g, dtype=torch.float32) * 2.0 - 1.0) * bound).to(t.dtype))
