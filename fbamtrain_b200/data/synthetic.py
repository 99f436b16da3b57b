"""Vectorised synthetic batch source for benchmarks and smoke runs.

Produces whole training batches with the statistics the benchmark configurations prescribe:
frames are ``rows x cols`` grids of cell ids drawn uniformly from ``[0, cell_vocab)`` (plus a
uniform colour-attribute id in ``[0, 16)`` mapped through the ANSI palette to fg/bg RGB); every
later frame copies its predecessor and redraws ``resample`` (5 %) of the cells; the target action
of each frame is uniform in ``[0, action_vocab)``.  Output lives in *pinned host memory* in the
cell-state layout the model consumes — ``uint32 (B, T, rows*cols, 3)`` — so a training step can
upload it with one asynchronous copy.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .palette import ANSI_PALETTE


class SyntheticBatchSource:
    def __init__(self, rows: int, cols: int, cell_vocab: int, action_vocab: int, seed: int = 0,
                 resample: float = 0.05, attr_ids: int = 16, pin: bool = True, native: Optional[bool] = None):
        """``native``: generate with the multi-threaded generator of the runtime library (default when it is built;
        ~50x faster than the NumPy loop, which otherwise takes longer than a training step).  The two generators
        follow the same recipe with different random streams, so their batches differ; each is reproducible from
        ``(seed, call number)``."""
        if native is None:
            from .. import runtime
            native = runtime.available()
        self.native = native
        self.rows, self.cols = rows, cols
        self.cell_vocab, self.action_vocab = cell_vocab, action_vocab
        self.resample, self.attr_ids = resample, attr_ids
        self.seed = seed
        self.pin = pin and torch.cuda.is_available()
        self._calls = 0

    def seek(self, call: int) -> None:
        """The next batch will be the one of call number ``call`` (batches are a function of seed and call number),
        e.g. the step count after resuming from a checkpoint."""
        self._calls = int(call)

    def next_batch(self, batch: int, seq: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(cells uint32-as-int32 (B, T, P, 3), targets int64 (B, T))`` on the host."""
        if self.native:
            from .. import runtime
            n = self.rows * self.cols
            cells = torch.empty((batch, seq, n, 3), dtype=torch.int32, pin_memory=self.pin)
            tg = torch.empty((batch, seq), dtype=torch.int64, pin_memory=self.pin)
            runtime.synth_fill(self.seed, self._calls, n, self.cell_vocab, self.attr_ids,
                               max(1, int(round(self.resample * n))), self.action_vocab, ANSI_PALETTE, cells, tg)
            self._calls += 1
            return cells, tg
        rng = np.random.default_rng([self.seed, self._calls])
        self._calls += 1
        n = self.rows * self.cols
        pal = np.asarray(ANSI_PALETTE, dtype=np.uint32)
        cp = rng.integers(0, self.cell_vocab, size=(batch, n), dtype=np.uint32)
        attr = rng.integers(0, self.attr_ids, size=(batch, n), dtype=np.uint32)
        k = max(1, int(round(self.resample * n)))
        cells = torch.empty((batch, seq, n, 3), dtype=torch.int32, pin_memory=self.pin)
        out = cells.numpy().view(np.uint32)
        rows_ix = np.arange(batch)[:, None]
        for t in range(seq):
            if t > 0:
                # k distinct cells per batch row: argpartition of random keys
                idx = np.argpartition(rng.random((batch, n), dtype=np.float32), k, axis=1)[:, :k]
                cp[rows_ix, idx] = rng.integers(0, self.cell_vocab, size=(batch, k), dtype=np.uint32)
                attr[rows_ix, idx] = rng.integers(0, self.attr_ids, size=(batch, k), dtype=np.uint32)
            out[:, t, :, 0] = cp
            out[:, t, :, 1] = pal[attr % 16]
            out[:, t, :, 2] = pal[(15 - attr) % 16]
        tg = torch.from_numpy(rng.integers(0, self.action_vocab, size=(batch, seq), dtype=np.int64))
        if self.pin:
            tg = tg.pin_memory()
        return cells, tg


class PrefetchingSource:
    """Generates the next batch of a source on a background thread while the current one trains (one batch ahead,
    same order as calling the source directly).  Generating an 8 x 1024-frame batch takes longer on a few host
    cores than a training step takes on the GPU; without this the loop would wait for its data."""

    def __init__(self, source, batch: int, seq: int):
        import queue
        import threading
        self.source, self.batch, self.seq = source, batch, seq
        self._queue: "queue.Queue" = queue.Queue(maxsize=1)
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._produce, name="fbam-synthetic-prefetch", daemon=True)
        self._thread.start()

    def _produce(self) -> None:
        import queue
        while not self._stop.is_set():
            try:
                item = self.source.next_batch(self.batch, self.seq)
            except BaseException as e:  # noqa: BLE001 - handed to the consumer
                item = e
            while not self._stop.is_set():
                try:
                    self._queue.put(item, timeout=0.1)
                    break
                except queue.Full:
                    continue
            if isinstance(item, BaseException):
                return

    def next_batch(self, batch: int, seq: int):
        if (batch, seq) != (self.batch, self.seq):
            raise ValueError("the prefetching source was set up for another batch shape")
        item = self._queue.get()
        if isinstance(item, BaseException):
            raise item
        return item

    def close(self) -> None:
        self._stop.set()
        try:
            self._queue.get_nowait()
        except Exception:  # noqa: BLE001 - empty queue
            pass
        self._thread.join(5)
