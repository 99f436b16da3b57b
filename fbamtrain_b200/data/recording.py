"""Recordings: sequences of terminal frames with the keystrokes typed while each frame was shown.

The reference reads ``.texz`` streams through the external ``termstreamxz`` library, which is not
part of its source tree (reference: ``src/dataset_iterator.cpp:218-266``).  Here a recording is an
interface; decoders are registered per file extension, and two implementations ship:

* :class:`ArrayRecording` — frames held in a NumPy array, loadable from ``.npz`` (extension
  ``.fbrec.npz``), used by tests and small experiments;
* :class:`RawRecording` — the uncompressed, memory-mapped ``.fbrec`` form that the native batch loader
  (``csrc/runtime/loader.cpp``) gathers from with worker threads;
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


RAW_MAGIC = b"FBAMREC1"
RAW_HEADER_BYTES = 64


def write_raw_recording(path: str, cells: np.ndarray, user_data: List[str]) -> None:
    """Writes the uncompressed, memory-mappable ``.fbrec`` form that the native batch loader gathers from:
    64-byte header (magic, rows, cols, frames, offset of the keystroke section), the ``uint32`` cell states, then
    ``frames + 1`` byte offsets into the UTF-8 keystroke blob that follows them."""
    cells = np.ascontiguousarray(cells, dtype=np.uint32)
    if cells.ndim != 4 or cells.shape[-1] != 3 or len(user_data) != cells.shape[0]:
        raise ValueError("cells must be (frames, rows, cols, 3) with one keystroke string per frame")
    frames, rows, cols = int(cells.shape[0]), int(cells.shape[1]), int(cells.shape[2])
    blobs = [u.encode("utf-8") for u in user_data]
    offsets = np.zeros(frames + 1, dtype=np.uint64)
    offsets[1:] = np.cumsum([len(b) for b in blobs], dtype=np.uint64)
    keys_offset = RAW_HEADER_BYTES + cells.nbytes
    header = RAW_MAGIC + np.array([rows, cols], dtype="<u4").tobytes() + \
        np.array([frames, keys_offset], dtype="<u8").tobytes()
    header += b"\0" * (RAW_HEADER_BYTES - len(header))
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(header)
        f.write(cells.tobytes())
        f.write(offsets.astype("<u8").tobytes())
        f.write(b"".join(blobs))
    os.replace(tmp, path)


class RawRecording(Recording):
    """A ``.fbrec`` file, memory-mapped (see :func:`write_raw_recording`)."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(RAW_HEADER_BYTES)
        if len(head) < RAW_HEADER_BYTES or head[:8] != RAW_MAGIC:
            raise ValueError(f"{path} is not a raw recording")
        self.rows, self.cols = (int(v) for v in np.frombuffer(head, dtype="<u4", count=2, offset=8))
        frames, keys_offset = (int(v) for v in np.frombuffer(head, dtype="<u8", count=2, offset=16))
        self._frames = frames
        self._cells = np.memmap(path, dtype="<u4", mode="r", offset=RAW_HEADER_BYTES,
                                shape=(frames, self.rows, self.cols, 3))
        self._offsets = np.memmap(path, dtype="<u8", mode="r", offset=keys_offset, shape=(frames + 1,))
        self._blob_base = keys_offset + (frames + 1) * 8
        self._blob = np.memmap(path, dtype=np.uint8, mode="r", offset=self._blob_base) \
            if int(self._offsets[-1]) > 0 else np.zeros(0, dtype=np.uint8)

    def total_frames(self) -> int:
        return self._frames

    def frame(self, index: int) -> Tuple[np.ndarray, str]:
        lo, hi = int(self._offsets[index]), int(self._offsets[index + 1])
        return self._cells[index], bytes(self._blob[lo:hi]).decode("utf-8")


_DECODERS: Dict[str, Callable[[str], Recording]] = {".fbrec.npz": ArrayRecording.load, ".fbrec": RawRecording}


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
