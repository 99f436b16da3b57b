"""Per-device stream bundle and allocator metrics.

The reference keeps, per device, a bundle of named streams — main, host→device, device→host, cleanup and numbered
compute streams with priorities (reference: ``tensorlib/include/gpu_stream.h:22-93``, ``stream_descriptor.h:7-64``) —
and reports allocator counters every step (reference: ``src/main.cpp:3803-3817``).  ``GpuStreamBundle`` is the same
idea on PyTorch streams: the trainer uploads on ``h2d``, the loss ring reads back on ``d2h``, the fused
data-parallel kernels of the action-model buckets run on ``compute(1)`` beside the frame head's backward.
``allocator_metrics`` returns peak / current / cached / reserved bytes of the caching allocator.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

_bundles: Dict[int, "GpuStreamBundle"] = {}


class GpuStreamBundle:
    def __init__(self, device: torch.device):
        self.device = device
        self.main = torch.cuda.current_stream(device)
        self.h2d = torch.cuda.Stream(device=device)
        self.d2h = torch.cuda.Stream(device=device)
        self.cleanup = torch.cuda.Stream(device=device, priority=0)
        self._compute: Dict[int, torch.cuda.Stream] = {}

    def compute(self, index: int, high_priority: bool = False) -> torch.cuda.Stream:
        if index not in self._compute:
            self._compute[index] = torch.cuda.Stream(device=self.device, priority=-1 if high_priority else 0)
        return self._compute[index]

    def wait_main(self, stream: torch.cuda.Stream) -> None:
        """``stream`` waits for everything queued on the main stream so far."""
        stream.wait_stream(torch.cuda.current_stream(self.device))

    def join(self, stream: torch.cuda.Stream) -> None:
        """The main stream waits for ``stream``."""
        torch.cuda.current_stream(self.device).wait_stream(stream)

    def synchronize(self) -> None:
        for s in [self.h2d, self.d2h, self.cleanup, *self._compute.values()]:
            s.synchronize()
        torch.cuda.current_stream(self.device).synchronize()


def stream_bundle(device: torch.device) -> Optional[GpuStreamBundle]:
    if device.type != "cuda":
        return None
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _bundles:
        _bundles[idx] = GpuStreamBundle(torch.device("cuda", idx))
    return _bundles[idx]


def allocator_metrics(device: torch.device) -> Dict[str, int]:
    if device.type != "cuda":
        return {"peak_bytes": 0, "current_bytes": 0, "cached_bytes": 0, "reserved_bytes": 0}
    s = torch.cuda.memory_stats(device)
    return {"peak_bytes": int(s.get("allocated_bytes.all.peak", 0)),
            "current_bytes": int(s.get("allocated_bytes.all.current", 0)),
            "cached_bytes": int(s.get("reserved_bytes.all.current", 0) - s.get("allocated_bytes.all.current", 0)),
            "reserved_bytes": int(s.get("reserved_bytes.all.current", 0))}
