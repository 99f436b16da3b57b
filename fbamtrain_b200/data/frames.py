"""Frame -> cell-state packing and keystroke -> action-token extraction.

Cell states are ``uint32 (batch, rows*cols, 3)``: channel 0 is the code point clamped to
``max_code_point - 1``, channels 1 and 2 are foreground / background packed ``r<<16 | g<<8 | b``
(reference: ``src/frame_utils.cpp:5-32``).

Action targets come from the keystrokes attached to frames: the stream is scanned with the trie
tokenizer, greedily taking the longest token; each token is paired with the frame that was on
screen when its first keystroke was typed (reference: ``src/main.cpp:1912-1981``).  A stream that
runs out of frames yields zero frames with target 0 (reference: ``src/main.cpp:1812-1884``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np

from ..tokenizer import Tokenizer
from .recording import Recording


def pack_rgb(r: int, g: int, b: int) -> int:
    return ((r & 0xFF) << 16) | ((g & 0xFF) << 8) | (b & 0xFF)


def prepare_cell_states(frame_cells: np.ndarray, max_code_point: int, out: Optional[np.ndarray] = None) -> np.ndarray:
    """Clamps code points and returns ``uint32 (rows*cols, 3)`` (written into ``out`` if given)."""
    flat = frame_cells.reshape(-1, 3)
    if out is None:
        out = np.empty_like(flat, dtype=np.uint32)
    np.minimum(flat[:, 0], np.uint32(max_code_point - 1), out=out[:, 0])
    out[:, 1] = flat[:, 1] & 0xFFFFFF
    out[:, 2] = flat[:, 2] & 0xFFFFFF
    return out


@dataclass
class StreamTokenizationContext:
    """Per-stream scanning state: position in the recording and keystrokes not yet consumed."""
    recording: Recording
    tokenizer: Tokenizer
    next_frame: int
    pending: List[Tuple[int, int]] = field(default_factory=list)  # (code point, frame index it was typed on)
    exhausted: bool = False

    def _fill(self) -> bool:
        """Appends the next frame's keystrokes; False when the recording has no more frames."""
        total = self.recording.total_frames()
        while self.next_frame < total:
            idx = self.next_frame
            self.next_frame += 1
            _, user = self.recording.frame(idx)
            if user:
                self.pending.extend((ord(ch), idx) for ch in user)
                return True
        return False


def consume_next_token(ctx: StreamTokenizationContext) -> Optional[Tuple[int, int]]:
    """Returns ``(token_id, frame_index_at_token_start)`` or None when the stream is exhausted."""
    while True:
        if not ctx.pending and not ctx._fill():
            return None
        handle = ctx.tokenizer.new_handle()
        best: Optional[Tuple[int, int]] = None  # (token id, code points consumed)
        i = 0
        while True:
            if i >= len(ctx.pending):
                # a longer token may continue into the next frame's keystrokes
                if not handle.has_continuation() or not ctx._fill():
                    break
            handle.add_char(ctx.pending[i][0])
            if handle.is_dead():
                break
            i += 1
            tid = handle.current_token_id()
            if tid is not None:
                best = (tid, i)
            if not handle.has_continuation():
                break
        if best is None:
            ctx.pending.pop(0)  # code point starts no token: skip it
            continue
        frame_idx = ctx.pending[0][1]
        del ctx.pending[: best[1]]
        return best[0], frame_idx
