"""SplitMix64 generator used for dataset iteration order.

Same sequence as the reference's ``Random`` (reference: ``src/random.cpp:9-25``): the state is
advanced by the 64-bit golden-ratio constant and mixed with two multiply/xor-shift rounds.
``randint`` reduces with a plain modulo, as the reference does, so cursors and checkpoints written
by either implementation resume to the same sample order.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


class SplitMix64:
    __slots__ = ("state",)

    def __init__(self, seed: int = 0):
        self.state = seed & _MASK

    def seed(self, seed: int) -> None:
        self.state = seed & _MASK

    def randu64(self) -> int:
        self.state = (self.state + _GOLDEN) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def randint(self, low: int, high: int) -> int:
        """Uniform-ish integer in [low, high) by modulo reduction."""
        if high <= low:
            raise ValueError("high must be > low")
        return low + self.randu64() % (high - low)
