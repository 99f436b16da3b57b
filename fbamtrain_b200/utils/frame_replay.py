"""Frame replay: the frames of a micro-batch stay in (pinned) host memory and only one chunk at a time is on the device.

The reference keeps its frame-head memory independent of the sequence length by re-decoding windows of 32 frames on a
CPU thread and running the frame head on them again in the backward (``src/main.cpp:1564, 1747-1792, 3354-3483``).
Here the decoded frames of the batch already sit in pinned host memory (the loader's output); :class:`FrameReplay`
uploads chunk ``i`` for the forward, and uploads it AGAIN for the backward, where :class:`ReplayedFrameHead` runs the
frame head on it a second time (not counted as useful FLOPs).  Two chunk-sized device buffers take turns and the
neighbouring chunk is copied on the host→device stream while the current one computes, in both directions (the last
two chunks of the forward are still in the buffers when the backward starts and are not copied again).  Device
memory for the frames and the frame head's activations is then one chunk's worth whatever B·T is.
"""
from __future__ import annotations

from typing import List, Optional

import torch


class FrameReplay:
    def __init__(self, host_cells: torch.Tensor, chunk: int, device: torch.device,
                 copy_stream: Optional["torch.cuda.Stream"] = None):
        """``host_cells``: ``(frames, P, 3)`` int32 on the host (pinned for asynchronous copies)."""
        self.host, self.chunk, self.device = host_cells, max(1, chunk), device
        self.frames = host_cells.shape[0]
        self.num_chunks = (self.frames + self.chunk - 1) // self.chunk
        self.cuda = device.type == "cuda"
        self.stream = copy_stream if self.cuda else None
        if self.cuda and self.stream is None:
            self.stream = torch.cuda.Stream(device=device)
        shape = (min(self.chunk, self.frames),) + tuple(host_cells.shape[1:])
        self.buffers = [torch.empty(shape, dtype=host_cells.dtype, device=device) for _ in range(2)] if self.cuda else []
        self.holds: List[Optional[int]] = [None, None]          # which chunk each buffer holds (or is receiving)
        self.ready: List[Optional["torch.cuda.Event"]] = [None, None]
        self.free: List[Optional["torch.cuda.Event"]] = [None, None]
        self.uploads = 0                                        # chunk copies issued (forward + replay)

    def bounds(self, i: int):
        lo = i * self.chunk
        return lo, min(self.frames, lo + self.chunk)

    def prefetch(self, i: int) -> None:
        """Starts the copy of chunk ``i`` into its buffer (``i`` outside the range: nothing)."""
        if not self.cuda or i < 0 or i >= self.num_chunks or self.holds[i & 1] == i:
            return
        slot = i & 1
        lo, hi = self.bounds(i)
        if self.free[slot] is not None:
            self.stream.wait_event(self.free[slot])            # the last reader of the buffer is done
        else:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            self.buffers[slot][:hi - lo].copy_(self.host[lo:hi], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        self.holds[slot], self.ready[slot] = i, ev
        self.uploads += 1

    def get(self, i: int) -> torch.Tensor:
        """Chunk ``i`` on the device; the compute stream waits for its copy."""
        lo, hi = self.bounds(i)
        if not self.cuda:
            self.uploads += 1
            return self.host[lo:hi].to(self.device)
        self.prefetch(i)
        slot = i & 1
        torch.cuda.current_stream(self.device).wait_event(self.ready[slot])
        return self.buffers[slot][:hi - lo]

    def release(self, i: int) -> None:
        """The compute stream is done reading chunk ``i`` (as far as it has been queued)."""
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record()
            self.free[i & 1] = ev


class ReplayedFrameHead(torch.autograd.Function):
    """Frame head on chunk ``i`` of a :class:`FrameReplay`: nothing of the chunk is kept for the backward, which
    fetches the chunk again, recomputes and back-propagates into the parameters' ``.grad``.  ``anchor`` is any
    tensor that requires grad (it ties the output into the autograd graph; it receives no gradient from here)."""

    @staticmethod
    def forward(ctx, anchor, frame_head, replay: FrameReplay, i: int):
        replay.prefetch(i + 1)
        cells = replay.get(i)
        with torch.no_grad():
            emb = frame_head(cells)
        replay.release(i)
        ctx.frame_head, ctx.replay, ctx.index = frame_head, replay, i
        return emb

    @staticmethod
    def backward(ctx, d_emb):
        from . import flops
        replay, i = ctx.replay, ctx.index
        replay.prefetch(i - 1)                                  # the backward walks the chunks downwards
        cells = replay.get(i)
        with torch.enable_grad(), flops.not_useful():
            emb = ctx.frame_head(cells)
        torch.autograd.backward(emb, d_emb)
        replay.release(i)
        return None, None, None, None
