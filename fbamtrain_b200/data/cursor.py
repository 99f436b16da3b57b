"""Durable dataset cursor: a small JSON file that survives a crash between checkpoints.

Contents and protocol follow the reference (reference: ``src/dataset_cursor.cpp:25, 70-122,
161-264, 313-348``): ``{"version": 1, "step_count", "rng_state", "batch_size",
"sequence_length"}``; ``commit()`` never blocks the training loop — it publishes the newest
snapshot to a writer thread, which writes a temporary file, ``fsync``s it, renames it over the
target and ``fsync``s the directory.  Only the newest snapshot matters; intermediate ones may be
skipped.  The native runtime library provides the same writer in C++
(``fbam_cursor_*`` in ``csrc/runtime/runtime.cpp``); this module is its Python front end and portable fallback.
"""
from __future__ import annotations

import json
import os
import threading
from dataclasses import asdict, dataclass
from typing import Optional

CURSOR_VERSION = 1


@dataclass
class DatasetCursorSnapshot:
    step_count: int = 0
    rng_state: int = 0
    batch_size: int = 0
    sequence_length: int = 0


def serialize_cursor(s: DatasetCursorSnapshot) -> str:
    d = {"version": CURSOR_VERSION}
    d.update(asdict(s))
    return json.dumps(d, indent=2) + "\n"


def write_durable_file(path: str, text: str) -> None:
    directory = os.path.dirname(os.path.abspath(path))
    os.makedirs(directory, exist_ok=True)
    tmp = path + ".tmp"
    fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o644)
    try:
        data = text.encode("utf-8")
        off = 0
        while off < len(data):
            off += os.write(fd, data[off:])
        os.fsync(fd)
    finally:
        os.close(fd)
    os.replace(tmp, path)
    dfd = os.open(directory, os.O_RDONLY)
    try:
        os.fsync(dfd)
    finally:
        os.close(dfd)


class DatasetCursorCommitter:
    def __init__(self, file_path: str):
        self.file_path = file_path
        self._lock = threading.Lock()
        self._cv = threading.Condition(self._lock)
        self._pending: Optional[DatasetCursorSnapshot] = None
        self._generation = 0
        self._written_generation = 0
        self._stop = False
        self._thread = threading.Thread(target=self._loop, name="fbam-cursor-writer", daemon=True)
        self._thread.start()

    @staticmethod
    def load(file_path: str) -> Optional[DatasetCursorSnapshot]:
        """Returns the stored snapshot, or None when the file is absent.  Raises on a malformed file."""
        if not file_path or not os.path.exists(file_path):
            return None
        with open(file_path, "r", encoding="utf-8") as f:
            d = json.load(f)
        if not isinstance(d, dict) or d.get("version") != CURSOR_VERSION:
            raise RuntimeError(f"Unsupported dataset cursor version in {file_path}")
        try:
            return DatasetCursorSnapshot(int(d["step_count"]), int(d["rng_state"]), int(d["batch_size"]),
                                         int(d["sequence_length"]))
        except KeyError as ex:
            raise RuntimeError(f"Dataset cursor {file_path} lacks field {ex}") from ex

    def commit(self, snapshot: DatasetCursorSnapshot) -> None:
        with self._lock:
            self._pending = snapshot
            self._generation += 1
            self._cv.notify_all()

    def flush(self, timeout: float = 10.0) -> bool:
        """Blocks until the newest committed snapshot is on disk."""
        with self._lock:
            target = self._generation
            return self._cv.wait_for(lambda: self._written_generation >= target, timeout)

    def _loop(self) -> None:
        while True:
            with self._lock:
                self._cv.wait_for(lambda: self._stop or self._generation != self._written_generation)
                if self._generation == self._written_generation and self._stop:
                    return
                snap, gen = self._pending, self._generation
            try:
                write_durable_file(self.file_path, serialize_cursor(snap))
            except OSError as ex:
                from ..utils.logging import LOG
                LOG("ERR", f"Failed to commit dataset cursor: {ex}")
            with self._lock:
                self._written_generation = gen
                self._cv.notify_all()

    def close(self) -> None:
        with self._lock:
            self._stop = True
            self._cv.notify_all()
        self._thread.join()
