"""The launch plan of a step: what ran, in which phase, with how many FLOPs.

There is no traced op graph in this package — a step is ordinary Python over persistent kernels — so the plan is
recorded, not built: inside :func:`record` every native entry point that launches kernels appends an entry (its
name, the enclosing phase range, the calling thread's role) and the FLOP accounting adds its count to the entry
that launched it.  The result answers what the reference's execution plan answers (reference:
``tensorlib/include/execution_plan.h:21-87`` — per-entry ``flop_estimate`` and ``is_useful``, ``totalFlops`` /
``totalUsefulFlops``; ``tensorlib/src/execution_backend.cpp:796-803`` — the launch log): the ordered kernel list
of one step, totals, and a per-kernel / per-phase summary.

``FBAMTRAIN_DUMP_PLAN=<file>`` makes the trainer record its first step and write the listing there.
"""
from __future__ import annotations

import contextlib
import threading
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Tuple


@dataclass
class PlanEntry:
    index: int
    name: str            # native entry point, e.g. fbam_gemm
    phase: str           # innermost phase range open on the launching thread ("" outside any)
    backward: bool       # launched from an autograd worker thread
    flops: float = 0.0
    useful_flops: float = 0.0


class StepPlan:
    def __init__(self) -> None:
        self.entries: List[PlanEntry] = []
        self._lock = threading.Lock()
        self._last = threading.local()          # the entry FLOPs reported on this thread belong to
        self._main_thread = threading.get_ident()

    # -- recording hooks -------------------------------------------------------------------------------------
    def on_launch(self, name: str) -> None:
        stack = getattr(_phase, "stack", None)
        entry = PlanEntry(0, name, stack[-1] if stack else "", threading.get_ident() != self._main_thread)
        with self._lock:
            entry.index = len(self.entries)
            self.entries.append(entry)
        self._last.entry = entry

    def on_flops(self, flops: float, useful: bool) -> None:
        entry = getattr(self._last, "entry", None)
        if entry is None:
            return
        entry.flops += flops
        if useful:
            entry.useful_flops += flops

    # -- queries ---------------------------------------------------------------------------------------------
    def total_flops(self) -> float:
        return sum(e.flops for e in self.entries)

    def total_useful_flops(self) -> float:
        return sum(e.useful_flops for e in self.entries)

    def by(self, field: str) -> Dict[str, Tuple[int, float]]:
        """``{name or phase: (launches, FLOPs)}``."""
        out: Dict[str, Tuple[int, float]] = {}
        for e in self.entries:
            key = getattr(e, field)
            n, f = out.get(key, (0, 0.0))
            out[key] = (n + 1, f + e.flops)
        return out

    def listing(self) -> str:
        lines = [f"# {len(self.entries)} launches, {self.total_flops() / 1e12:.3f} TFLOP "
                 f"({self.total_useful_flops() / 1e12:.3f} useful)"]
        for e in self.entries:
            flops = f"{e.flops / 1e9:12.3f} GFLOP" + ("" if e.useful_flops == e.flops else " (recompute)") \
                if e.flops else " " * 18
            lines.append(f"{e.index:5d}  {'bwd' if e.backward else 'fwd'}  {e.name:<28s} {flops}  {e.phase}")
        lines.append("# by kernel")
        for name, (n, f) in sorted(self.by("name").items(), key=lambda kv: -kv[1][1]):
            lines.append(f"#   {name:<28s} x{n:<5d} {f / 1e12:9.3f} TFLOP")
        lines.append("# by phase")
        for name, (n, f) in sorted(self.by("phase").items(), key=lambda kv: -kv[1][1]):
            lines.append(f"#   {name or '-':<44s} x{n:<5d} {f / 1e12:9.3f} TFLOP")
        return "\n".join(lines) + "\n"


_active: Optional[StepPlan] = None
_phase = threading.local()


def active() -> Optional[StepPlan]:
    return _active


@contextlib.contextmanager
def record() -> Iterator[StepPlan]:
    """Records the native launches made inside the block (by any thread) into a :class:`StepPlan`."""
    global _active
    if _active is not None:
        raise RuntimeError("a plan is already being recorded")
    plan = StepPlan()
    _active = plan
    try:
        yield plan
    finally:
        _active = None


def push_phase(name: str) -> None:
    stack = getattr(_phase, "stack", None)
    if stack is None:
        stack = _phase.stack = []
    stack.append(name)


def pop_phase() -> None:
    _phase.stack.pop()
