"""Recordings: sequences of terminal frames with the keystrokes typed while each frame was shown.

The reference reads ``.texz`` streams through the external ``termstreamxz`` library, which is not
part of its source tree (reference: ``src/dataset_iterator.cpp:218-266``).  Here a recording is an
interface; decoders are registered per file extension, and two implementations ship:

* :class:`ArrayRecording` — frames held in a NumPy array, loadable from ``.npz`` (extension
  ``.fbrec.npz``), used by tests and small experiments;
* :class:`SyntheticRecording` — the seeded generator that the benchmark configurations specify:
  the first frame is uniform random, every later frame copies its predecessor and resamples a
  fixed fraction of the cells.

A frame is ``uint32 (rows, cols, 3)``: code point, foreground ``0xRRGGBB``, background ``0xRRGGBB``
(reference: ``include/frame_utils.h:6-11``), plus a ``user_data`` string of keystrokes.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Tuple

import numpy as np

from .palette import ANSI_PALETTE


class Recording:
    """Random-access view of one recorded session."""

    rows: int
    cols: int

    def total_frames(self) -> int:
        raise NotImplementedError

    def frame(self, index: int) -> Tuple[np.ndarray, str]:
        """Returns ``(cells uint32 (rows, cols, 3), user_data)`` for frame ``index``."""
        raise NotImplementedError


class ArrayRecording(Recording):
    def __init__(self, cells: np.ndarray, user_data: List[str]):
        if cells.ndim != 4 or cells.shape[-1] != 3:
            raise ValueError("cells must have shape (frames, rows, cols, 3)")
        if len(user_data) != cells.shape[0]:
            raise ValueError("one user_data string per frame is required")
        self._cells = np.ascontiguousarray(cells, dtype=np.uint32)
        self._user = list(user_data)
        self.rows, self.cols = int(cells.shape[1]), int(cells.shape[2])

    def total_frames(self) -> int:
        return int(self._cells.shape[0])

    def frame(self, index: int) -> Tuple[np.ndarray, str]:
        return self._cells[index], self._user[index]

    def save(self, path: str) -> None:
        np.savez_compressed(path, cells=self._cells, user_data=np.array(self._user, dtype=object))

    @staticmethod
    def load(path: str) -> "ArrayRecording":
        with np.load(path, allow_pickle=True) as z:
            return ArrayRecording(z["cells"], [str(s) for s in z["user_data"]])


class SyntheticRecording(Recording):
    """Seeded synthetic session.  Frame 0 is uniform; frame t copies frame t-1 and redraws
    ``resample`` of its cells.  Each frame carries one keystroke drawn from ``alphabet``."""

    def __init__(self, rows: int, cols: int, frames: int, seed: int, cell_vocab: int = 256,
                 resample: float = 0.05, alphabet: str = "abcdefghijklmnopqrstuvwxyz", attr_ids: int = 16):
        self.rows, self.cols = rows, cols
        rng = np.random.default_rng(seed)
        n = rows * cols
        cp = rng.integers(0, cell_vocab, size=n, dtype=np.uint32)
        attr = rng.integers(0, attr_ids, size=n, dtype=np.uint32)
        cells = np.empty((frames, n, 3), dtype=np.uint32)
        k = max(1, int(round(resample * n)))
        pal = np.asarray(ANSI_PALETTE, dtype=np.uint32)
        for t in range(frames):
            if t > 0:
                idx = rng.choice(n, size=k, replace=False)
                cp[idx] = rng.integers(0, cell_vocab, size=k, dtype=np.uint32)
                attr[idx] = rng.integers(0, attr_ids, size=k, dtype=np.uint32)
            cells[t, :, 0] = cp
            cells[t, :, 1] = pal[attr % 16]
            cells[t, :, 2] = pal[(15 - attr) % 16]
        self._cells = cells.reshape(frames, rows, cols, 3)
        keys = rng.integers(0, len(alphabet), size=frames)
        self._user = [alphabet[int(i)] for i in keys]

    def total_frames(self) -> int:
        return int(self._cells.shape[0])

    def frame(self, index: int) -> Tuple[np.ndarray, str]:
        return self._cells[index], self._user[index]


_DECODERS: Dict[str, Callable[[str], Recording]] = {".fbrec.npz": ArrayRecording.load}


def register_decoder(extension: str, factory: Callable[[str], Recording]) -> None:
    """Registers a decoder for files ending in ``extension`` (e.g. ``".texz"``)."""
    _DECODERS[extension] = factory


def recording_extensions() -> List[str]:
    return list(_DECODERS)


def open_recording(path: str) -> Recording:
    for ext, factory in _DECODERS.items():
        if path.endswith(ext):
            return factory(path)
    raise ValueError(f"No decoder registered for recording '{os.path.basename(path)}' "
                     f"(known extensions: {sorted(_DECODERS)})")
