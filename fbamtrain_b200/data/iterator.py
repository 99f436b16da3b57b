"""Seeded on-the-fly dataset iteration with a background prefetch thread.

Behaviour follows the reference iterator (reference: ``src/dataset_iterator.cpp:144-201, 218-405``):

* recordings are the files of one directory, sorted by path;
* nothing is shuffled up front — for every batch item the SplitMix64 stream yields
  ``file = rand % n_files`` and then ``start = rand % (max(0, frames - seq_len) + 1)``;
* a worker thread prepares batch *k+1* while batch *k* is consumed (two buffers, alternating);
* ``checkpoint()`` captures the RNG state *after* the prepared batch was drawn together with the
  prepared indices/starts and the buffer index, so a restore replays exactly that batch;
  ``cursor_checkpoint()`` captures only the RNG state of the batch most recently handed out;
  ``restore()`` accepts either form (RNG-only states trigger a fresh draw).
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..rng import SplitMix64
from .recording import Recording, open_recording, recording_extensions


@dataclass
class DatasetIteratorState:
    rng_state: int = 0
    batch_size: int = 0
    prefetch_buffer_index: int = 0
    prepared_indices: List[int] = field(default_factory=list)
    prepared_start_positions: List[int] = field(default_factory=list)


@dataclass
class Batch:
    """One batch: per item, the recording and the frame index where its sequence starts; ``tensors`` holds what
    the iterator's assembler produced for it on the prefetch thread (None without an assembler)."""
    recordings: List[Recording]
    indices: List[int]
    start_positions: List[int]
    tensors: Optional[object] = None


class RecordingDatasetIterator:
    def __init__(self, recordings_folder_path: Optional[str], batch_size: int, sequence_length: int, seed: int,
                 recordings: Optional[Sequence[Recording]] = None,
                 assembler: Optional[Callable[[List[int], List[int], int], object]] = None):
        """``assembler(indices, start_positions, buffer_index)`` — optional; called on the prefetch thread for every
        prepared batch (outside the iterator's lock), its result travels with the batch.  ``buffer_index``
        alternates between 0 and 1 so the assembler can fill two (pinned) buffers in turn: the one handed out with
        batch k stays untouched until batch k + 2 is prepared."""
        self._assembler = assembler
        self._prepared_tensors = None
        self.batch_size, self.sequence_length, self.seed = int(batch_size), int(sequence_length), int(seed)
        if recordings is not None:
            self._recordings: List[Optional[Recording]] = list(recordings)
            self._paths = [f"<memory:{i}>" for i in range(len(self._recordings))]
        else:
            if recordings_folder_path is None or not os.path.isdir(recordings_folder_path):
                raise RuntimeError(
                    f"Recordings folder path does not exist or is not a directory: {recordings_folder_path}")
            exts = tuple(recording_extensions())
            self._paths = sorted(os.path.join(recordings_folder_path, f) for f in os.listdir(recordings_folder_path)
                                 if f.endswith(exts) and not os.path.isdir(os.path.join(recordings_folder_path, f)))
            if not self._paths:
                raise RuntimeError(f"No recordings found in folder: {recordings_folder_path}")
            self._recordings = [open_recording(p) for p in self._paths]
        if not self._recordings:
            raise RuntimeError("No recordings available for dataset iterator.")
        self._total_frames = [r.total_frames() for r in self._recordings]

        self._rng = SplitMix64(seed)
        self._mutex = threading.Lock()
        self._cv_request = threading.Condition(self._mutex)
        self._cv_ready = threading.Condition(self._mutex)
        self._stop = False
        self._requested = False
        self._ready = False
        self._buffer_index = 0
        self._prepared_indices: List[int] = []
        self._prepared_starts: List[int] = []
        self._prepared_rng_state = self._rng.state
        self._cursor_rng_state = self._rng.state
        self._worker: Optional[threading.Thread] = None
        self._start_worker()
        self._request_prefetch()

    # -- worker -------------------------------------------------------------------------------
    def _draw(self):
        n = len(self._recordings)
        indices, starts = [], []
        for _ in range(self.batch_size):
            idx = self._rng.randint(0, n)
            total = self._total_frames[idx]
            max_start = max(0, total - self.sequence_length)
            start = 0 if total <= 0 else self._rng.randint(0, max_start + 1)
            indices.append(idx)
            starts.append(start)
        return indices, starts

    def _worker_loop(self) -> None:
        while True:
            with self._mutex:
                self._cv_request.wait_for(lambda: self._stop or self._requested)
                if self._stop:
                    return
                self._requested = False
                buf = self._buffer_index
                indices, starts = self._draw()          # only this thread touches the RNG while it runs
                rng_state = self._rng.state
            tensors = self._assembler(indices, starts, buf) if self._assembler is not None else None
            with self._mutex:
                if self._stop:
                    return
                self._prepared_indices, self._prepared_starts = indices, starts
                self._prepared_rng_state = rng_state
                self._prepared_tensors = tensors
                self._ready = True
                self._buffer_index = 1 - buf
                self._cv_ready.notify_all()

    def _start_worker(self) -> None:
        self._stop = False
        self._worker = threading.Thread(target=self._worker_loop, name="fbam-dataset-prefetch", daemon=True)
        self._worker.start()

    def _stop_worker(self) -> None:
        with self._mutex:
            self._stop = True
            self._cv_request.notify_all()
            self._cv_ready.notify_all()
        if self._worker is not None:
            self._worker.join()
            self._worker = None

    def _request_prefetch(self) -> None:
        with self._mutex:
            self._requested = True
            self._cv_request.notify_all()

    # -- public API ---------------------------------------------------------------------------
    def next_batch(self) -> Batch:
        with self._mutex:
            self._cv_ready.wait_for(lambda: self._ready or self._stop)
            if not self._ready:
                raise RuntimeError("Dataset iterator was stopped.")
            indices, starts = list(self._prepared_indices), list(self._prepared_starts)
            tensors, self._prepared_tensors = self._prepared_tensors, None
            buf = 1 - self._buffer_index               # the buffer the prepared batch was (or would be) written to
            self._cursor_rng_state = self._prepared_rng_state
            self._ready = False
            self._requested = True
            self._cv_request.notify_all()
        if tensors is None and self._assembler is not None:   # a batch restored from a checkpoint: assemble it now
            tensors = self._assembler(indices, starts, buf)
        return Batch([self._recordings[i] for i in indices], indices, starts, tensors)

    def cursor_checkpoint(self) -> DatasetIteratorState:
        return DatasetIteratorState(rng_state=self._cursor_rng_state, batch_size=self.batch_size,
                                    prefetch_buffer_index=0)

    def checkpoint(self) -> DatasetIteratorState:
        with self._mutex:
            self._cv_ready.wait_for(lambda: self._ready or self._stop)
            if not self._ready:
                raise RuntimeError("Dataset iterator has no prefetched batch to checkpoint.")
            return DatasetIteratorState(self._prepared_rng_state, self.batch_size, self._buffer_index,
                                        list(self._prepared_indices), list(self._prepared_starts))

    def restore(self, state: DatasetIteratorState) -> None:
        if state.batch_size != self.batch_size:
            raise RuntimeError("Checkpoint batch size does not match dataset iterator batch size.")
        if state.prefetch_buffer_index > 1:
            raise RuntimeError("Checkpoint prefetch_buffer_index must be 0 or 1.")
        has_idx, has_start = bool(state.prepared_indices), bool(state.prepared_start_positions)
        if has_idx != has_start:
            raise RuntimeError("Checkpoint prefetch state is incomplete.")
        if has_idx:
            if len(state.prepared_indices) != self.batch_size:
                raise RuntimeError("Checkpoint prepared_indices size mismatch.")
            if len(state.prepared_start_positions) != self.batch_size:
                raise RuntimeError("Checkpoint prepared_start_positions size mismatch.")
            if any(i >= len(self._recordings) for i in state.prepared_indices):
                raise RuntimeError("Checkpoint file index out of range for dataset iterator.")
        self._stop_worker()
        with self._mutex:
            self._requested = False
            self._ready = has_idx
            self._buffer_index = state.prefetch_buffer_index
            self._prepared_indices = list(state.prepared_indices)
            self._prepared_starts = list(state.prepared_start_positions)
            self._prepared_rng_state = state.rng_state
            self._prepared_tensors = None
            self._cursor_rng_state = state.rng_state
            self._rng.state = state.rng_state
        self._start_worker()
        if not has_idx:
            self._request_prefetch()

    def close(self) -> None:
        self._stop_worker()

    def __del__(self):  # best effort; the worker is a daemon thread
        try:
            self._stop_worker()
        except Exception:  # noqa: BLE001
            pass
