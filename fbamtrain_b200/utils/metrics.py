"""Step metrics without host synchronisation in the training loop.

``LossRingBuffer`` keeps 128 device scalars; micro-batch losses are added on the device, and when a
step is finalised its slot is copied to pinned host memory on a side stream behind an event.
``AsyncStepLogger`` is a thread that consumes finished steps: it waits on the step's end event,
reads the loss slot, and emits ``Step N took s seconds; seqlen/time = …; loss/train = …`` plus — when
``FBAMTRAIN_METRICS_JSON`` is set — one JSON object per line
(``{"step": N, "step_time_sec": …, "loss/train": …}``; validation lines use ``loss/validation``).
Dropped steps discard their slot.  (reference: ``src/loss_accumulation_ring_buffer.cpp:67-189``,
``src/async_step_logger.cpp:71-186``, ``include/async_step_logger.h:15-123``.)
"""
from __future__ import annotations

import json
import os
import queue
import sys
import threading
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch

from .logging import LOG

RING_SLOTS = 128


class LossRingBuffer:
    def __init__(self, device: torch.device):
        self.device = device
        self.ring = torch.zeros(RING_SLOTS, dtype=torch.float32, device=device)
        self.host = torch.zeros(RING_SLOTS, dtype=torch.float32)
        self.cuda = device.type == "cuda"
        if self.cuda:
            from .streams import stream_bundle
            self.host = self.host.pin_memory()
            self.d2h = stream_bundle(device).d2h

    def begin(self, step: int) -> None:
        self.ring[step % RING_SLOTS].zero_()

    def accumulate(self, step: int, loss: torch.Tensor) -> None:
        self.ring[step % RING_SLOTS].add_(loss.detach().float())

    def finalize(self, step: int):
        """Starts the device→host copy of the step's slot; returns an event to wait on (or None on CPU)."""
        slot = step % RING_SLOTS
        if not self.cuda:
            self.host[slot] = self.ring[slot]
            return None
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(ready)
            self.host[slot].copy_(self.ring[slot], non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        return done

    def read(self, step: int) -> float:
        return float(self.host[step % RING_SLOTS])


@dataclass
class StepRecord:
    step: int
    start_event: object
    end_event: object
    loss_event: object
    seq_len: int
    batch: int
    dropped: bool = False
    wall_start: float = 0.0
    wall_end: float = 0.0
    useful_flops: float = 0.0      # tensor-core FLOPs launched by this rank during the step, recomputation excluded
    total_flops: float = 0.0


@dataclass
class ProgressRecord:
    """``done`` of ``total`` frames of a phase have been processed once ``event`` completes; the rate is measured
    from ``phase_start`` (GPU events, or wall-clock seconds on CPU)."""
    label: str                 # "Sequence position" (forward) or "Backward sequence position"
    done: int
    total: int
    phase_start: object
    event: object


class AsyncStepLogger:
    def __init__(self, ring: LossRingBuffer, sink: Optional[Callable[[dict], None]] = None):
        self.ring = ring
        self.sink = sink
        self.json_lines = bool(os.environ.get("FBAMTRAIN_METRICS_JSON"))
        self.history: List[dict] = []
        self._q: "queue.Queue[Optional[StepRecord]]" = queue.Queue()
        self._thread = threading.Thread(target=self._loop, name="fbam-step-logger", daemon=True)
        self._thread.start()

    def submit(self, rec: StepRecord) -> None:
        self._q.put(rec)

    def progress(self, rec: ProgressRecord) -> None:
        """Queues a line ``<label> done/total processed | FPS: x`` (reference: ``src/async_step_logger.cpp:115-170``;
        FPS = frames processed / time since the phase began)."""
        self._q.put(rec)

    def _progress_line(self, rec: ProgressRecord) -> None:
        if isinstance(rec.event, float):
            seconds = rec.event - rec.phase_start
        else:
            rec.event.synchronize()
            seconds = rec.phase_start.elapsed_time(rec.event) / 1e3
        fps = rec.done / seconds if seconds > 0 else float("inf")
        LOG("INFO", f"{rec.label} {rec.done}/{rec.total} processed | FPS: {fps:.1f}")

    def log_validation(self, step: int, loss: float) -> None:
        LOG("INFO", f"Step {step} validation loss = {loss:.6f}")
        if self.json_lines:
            sys.stdout.write(json.dumps({"step": step, "loss/validation": loss}) + "\n")
            sys.stdout.flush()

    def _loop(self) -> None:
        while True:
            rec = self._q.get()
            if rec is None:
                return
            if isinstance(rec, ProgressRecord):
                try:
                    self._progress_line(rec)
                finally:
                    self._q.task_done()
                continue
            try:
                if rec.end_event is not None:
                    rec.end_event.synchronize()
                    seconds = rec.start_event.elapsed_time(rec.end_event) / 1e3
                else:
                    seconds = rec.wall_end - rec.wall_start
                if rec.dropped:
                    LOG("WARN", f"Step {rec.step} dropped after {seconds:.4f} seconds")
                    continue
                if rec.loss_event is not None:
                    rec.loss_event.synchronize()
                loss = self.ring.read(rec.step)
                rate = rec.seq_len * rec.batch / seconds if seconds > 0 else float("inf")
                entry = {"step": rec.step, "step_time_sec": seconds, "loss/train": loss, "frames_per_sec": rate}
                if rec.useful_flops > 0 and seconds > 0:
                    from .mfu import mfu as _mfu
                    entry["tflops_useful"] = rec.useful_flops / seconds / 1e12
                    entry["tflops_total"] = rec.total_flops / seconds / 1e12
                    entry["mfu"] = _mfu(rec.useful_flops, seconds)
                self.history.append(entry)
                LOG("INFO", f"Step {rec.step} took {seconds:.4f} seconds; seqlen/time = "
                            f"{rec.seq_len / seconds if seconds > 0 else float('inf'):.2f}; loss/train = {loss:.6f}")
                if self.json_lines:
                    line = {"step": rec.step, "step_time_sec": seconds, "loss/train": loss}
                    if "mfu" in entry:
                        line["mfu"] = entry["mfu"]
                    sys.stdout.write(json.dumps(line) + "\n")
                    sys.stdout.flush()
                if self.sink is not None:
                    self.sink(entry)
            finally:
                self._q.task_done()

    def drain(self) -> None:
        self._q.join()

    def close(self) -> None:
        self._q.put(None)
        self._thread.join()
