"""Chunked host↔device streaming of time-major tensors that live in pinned host memory.

``TensorStreamIterator`` walks dimension 0 of a pinned tensor in chunks and uploads chunk *k+1* on a copy stream
while chunk *k* is being consumed (double buffering); ``TensorStreamPopulator`` writes device chunks back to a
pinned tensor, optionally keeping only every ``interval``-th step (that is how the reference thins the LSTM cell
state into recompute checkpoints).  (reference: ``tensorlib/src/tensor_stream_iterator.cpp:8-114``,
``tensor_stream_populator.cpp:5-85``.)
"""
from __future__ import annotations

from typing import Iterator, Optional, Tuple

import torch


class TensorStreamIterator:
    def __init__(self, host: torch.Tensor, chunk: int, device: torch.device, reverse: bool = False,
                 stream: Optional[torch.cuda.Stream] = None):
        self.host, self.chunk, self.device, self.reverse = host, max(1, chunk), device, reverse
        self.cuda = device.type == "cuda" and not host.is_cuda
        self.stream = stream or (torch.cuda.Stream(device=device) if self.cuda else None)
        n = host.shape[0]
        bounds = [(lo, min(n, lo + self.chunk)) for lo in range(0, n, self.chunk)]
        self.bounds = bounds[::-1] if reverse else bounds

    def _start(self, lo: int, hi: int):
        src = self.host[lo:hi]
        if not self.cuda:
            return src.to(self.device), None
        buf = torch.empty(src.shape, dtype=src.dtype, device=self.device)
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            buf.copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        return buf, ev

    def __iter__(self) -> Iterator[Tuple[int, int, torch.Tensor]]:
        pending = self._start(*self.bounds[0]) if self.bounds else None
        for i, (lo, hi) in enumerate(self.bounds):
            buf, ev = pending
            pending = self._start(*self.bounds[i + 1]) if i + 1 < len(self.bounds) else None   # prefetch
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
                buf.record_stream(torch.cuda.current_stream())
            yield lo, hi, buf


class TensorStreamPopulator:
    def __init__(self, host: torch.Tensor, interval: int = 1, stream: Optional[torch.cuda.Stream] = None):
        self.host, self.interval = host, max(1, interval)
        self.stream = stream
        self._events = []

    def write(self, lo: int, chunk: torch.Tensor) -> None:
        """``chunk`` holds steps ``lo .. lo+len``; step ``t`` lands in row ``t // interval`` when ``t % interval == 0``."""
        n = chunk.shape[0]
        if self.interval == 1:
            rows_src, row0 = chunk, lo
        else:
            first = (-lo) % self.interval
            rows_src, row0 = chunk[first::self.interval], (lo + first) // self.interval
        if rows_src.shape[0] == 0:
            return
        dst = self.host[row0:row0 + rows_src.shape[0]]
        if not chunk.is_cuda:
            dst.copy_(rows_src)
            return
        stream = self.stream or torch.cuda.current_stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            dst.copy_(rows_src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        rows_src.record_stream(stream)
        self._events.append(ev)

    def synchronize(self) -> None:
        for ev in self._events:
            ev.synchronize()
        self._events.clear()
