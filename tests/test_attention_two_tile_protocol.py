"""Randomised-schedule model of the barrier protocol of the two-tile attention forward (``attn_fwd2_kernel`` in
``csrc/attention_tcgen05.cu``): one MMA / TMA issuing thread and two softmax groups that share each K and V block.

The model follows the kernel's order of waits, loads, MMAs and commits one for one (mbarrier parities included: a
wait succeeds when the barrier's completed-phase count has the other parity) and runs it under random latencies
of loads, MMAs and softmax work.  It checks what the kernel's correctness rests on: no deadlock, no K or V block
overwritten before the MMAs that read it have completed, no S or O accumulator overwritten before its softmax
group has read it, no P tile overwritten before the P·V product that reads it has completed, and every MMA
issued with the operands of the block it belongs to.  A protocol change in the kernel has to be made here too.
"""
import random

import pytest


class Barrier:
    """An mbarrier: ``need`` arrivals complete a phase; ``test(parity)`` is ``mbarrier.try_wait.parity``."""

    def __init__(self, need: int = 1):
        self.need, self.arrived, self.completions = need, 0, 0

    def arrive(self) -> None:
        self.arrived += 1
        if self.arrived == self.need:
            self.arrived = 0
            self.completions += 1

    def test(self, parity: int) -> bool:
        return (self.completions & 1) != parity


class Simulation:
    """State shared by the three agents plus the event queue of asynchronous completions."""

    def __init__(self, blocks_per_tile, seed: int, skip_k_empty_wait: bool = False):
        self.rnd = random.Random(seed)
        self.nk = list(blocks_per_tile)                  # key blocks tile 0 / tile 1 attends to (causal: differ)
        self.nkb = max(self.nk)
        self.skip_k_empty_wait = skip_k_empty_wait       # fault injection for the self-test of the model
        names = ["k_full", "k_empty", "v_full", "v_empty"] + [f"{n}{g}" for n in ("s_full", "p_ready", "pv_full")
                                                                for g in range(2)]
        self.bars = {n: Barrier() for n in names}        # a softmax group is modelled as one arriving agent
        self.now = 0.0
        self.mma_busy_until = 0.0
        self.pending = []                                # (time, tie-break, action)
        self.errors = []
        self.k_in_smem = self.v_in_smem = -1
        self.s_block = [-1, -1]                          # block whose S / O / P currently sits in TMEM / smem
        self.o_block = [-1, -1]
        self.p_block = [-1, -1]
        self.s_read = [-1, -1]                           # last block whose S / O the softmax group has read
        self.o_read = [-1, -1]
        self.s_done = [-1, -1]                           # last block whose S / P·V MMAs have completed
        self.pv_done = [-1, -1]

    def at(self, time: float, action) -> None:
        self.pending.append((time, self.rnd.random(), action))

    # -- what the issuing thread does ------------------------------------------------------------------------
    def load(self, kind: str, kb: int) -> None:
        done = self.s_done if kind == "k" else self.pv_done
        for g in range(2):
            if 0 <= kb - 1 < self.nk[g] and done[g] < kb - 1:
                self.errors.append(f"{kind.upper()} block {kb - 1} overwritten before tile {g}'s MMAs read it")

        def landed():
            if kind == "k":
                self.k_in_smem = kb
            else:
                self.v_in_smem = kb
            self.bars[f"{kind}_full"].arrive()
        self.at(self.now + self.rnd.uniform(0.5, 3.0), landed)

    def issue(self, kind: str, g: int, kb: int) -> None:
        start = max(self.now, self.mma_busy_until)
        end = start + self.rnd.uniform(0.2, 1.0)
        self.mma_busy_until = end
        if kind == "s":
            if self.k_in_smem != kb:
                self.errors.append(f"S{g}({kb}) issued while K holds block {self.k_in_smem}")
            if self.s_read[g] < kb - 1:
                self.errors.append(f"S{g}({kb}) overwrites S({kb - 1}) before it was read")

            def done():
                self.s_block[g] = self.s_done[g] = kb
        else:
            if self.v_in_smem != kb:
                self.errors.append(f"PV{g}({kb}) issued while V holds block {self.v_in_smem}")
            if self.p_block[g] != kb:
                self.errors.append(f"PV{g}({kb}) issued while P holds block {self.p_block[g]}")
            if self.o_read[g] < kb - 1:
                self.errors.append(f"PV{g}({kb}) overwrites O({kb - 1}) before it was read")

            def done():
                self.o_block[g] = self.pv_done[g] = kb
        self.at(end, done)

    def commit(self, bar: str) -> None:
        """tcgen05.commit: the barrier is arrived on once everything issued so far has completed."""
        self.at(max(self.mma_busy_until, self.now) + 1e-6, self.bars[bar].arrive)

    # -- the agents (generators that yield what they wait for) -------------------------------------------------
    def mma_thread(self):
        nk, nkb = self.nk, self.nkb
        if nkb > 0:
            self.load("k", 0)
            self.load("v", 0)
            yield ("wait", "k_full", 0)                  # (the wait for Q is folded in)
            for g in range(2):
                if 0 < nk[g]:
                    self.issue("s", g, 0)
                    self.commit(f"s_full{g}")
            self.commit("k_empty")
        for kb in range(nkb):
            ph, more = kb & 1, kb + 1 < nkb
            if more:
                if not self.skip_k_empty_wait:
                    yield ("wait", "k_empty", ph)
                self.load("k", kb + 1)
            yield ("wait", "v_full", ph)
            if kb < nk[0]:
                yield ("wait", "p_ready0", ph)
                self.issue("pv", 0, kb)
                self.commit("pv_full0")
            if more:
                yield ("wait", "k_full", ph ^ 1)
                if kb + 1 < nk[0]:
                    self.issue("s", 0, kb + 1)
                    self.commit("s_full0")
            if kb < nk[1]:
                yield ("wait", "p_ready1", ph)
                self.issue("pv", 1, kb)
                self.commit("pv_full1")
            self.commit("v_empty")
            if more:
                if kb + 1 < nk[1]:
                    self.issue("s", 1, kb + 1)
                    self.commit("s_full1")
                self.commit("k_empty")
                yield ("wait", "v_empty", ph)
                self.load("v", kb + 1)

    def softmax_group(self, g: int):
        for kb in range(self.nk[g]):
            yield ("wait", f"s_full{g}", kb & 1)
            if self.s_block[g] != kb:
                self.errors.append(f"softmax {g} reads S of block {self.s_block[g]}, expected {kb}")
            yield ("sleep", self.rnd.uniform(0.3, 2.5))
            self.s_read[g] = kb
            if kb > 0 and self.pv_done[g] < kb - 1:
                self.errors.append(f"softmax {g} overwrites P({kb - 1}) before its P·V completed")
            self.p_block[g] = kb
            self.bars[f"p_ready{g}"].arrive()
            yield ("wait", f"pv_full{g}", kb & 1)
            if self.o_block[g] != kb:
                self.errors.append(f"softmax {g} reads O of block {self.o_block[g]}, expected {kb}")
            yield ("sleep", self.rnd.uniform(0.1, 0.8))
            self.o_read[g] = kb

    # -- scheduler -------------------------------------------------------------------------------------------
    def run(self):
        agents = {"mma": self.mma_thread(), "softmax0": self.softmax_group(0), "softmax1": self.softmax_group(1)}
        waiting, sleeping = {}, {}

        def advance(name):
            try:
                request = next(agents[name])
            except StopIteration:
                del agents[name]
                return
            if request[0] == "wait":
                waiting[name] = request[1:]
            else:
                sleeping[name] = self.now + request[1]

        for name in list(agents):
            advance(name)
        for _ in range(100000):
            if not agents:
                return self.errors
            ready = [n for n, (bar, parity) in waiting.items() if self.bars[bar].test(parity)]
            ready += [n for n, t in sleeping.items() if t <= self.now]
            if ready:
                for name in ready:
                    waiting.pop(name, None)
                    sleeping.pop(name, None)
                    advance(name)
                continue
            times = [t for t, _, _ in self.pending] + list(sleeping.values())
            if not times:
                counts = {k: b.completions for k, b in self.bars.items()}
                return self.errors + [f"deadlock: waiting {waiting}, completed phases {counts}"]
            self.now = min(times)
            due = sorted(p for p in self.pending if p[0] <= self.now)
            for item in due:
                self.pending.remove(item)
                item[2]()
        return self.errors + ["no progress"]


@pytest.mark.parametrize("blocks", [(1, 1), (2, 2), (3, 3), (8, 8), (1, 2), (3, 4), (7, 8), (2, 0), (5, 0), (1, 0), (4, 5)])
def test_two_tile_attention_protocol_has_no_deadlock_or_hazard(blocks):
    for seed in range(60):
        assert Simulation(blocks, seed).run() == [], (blocks, seed)


def test_the_model_notices_a_missing_wait():
    """The checks are live: without the wait that protects the K buffer an early overwrite is reported."""
    assert any(Simulation((3, 4), seed, skip_k_empty_wait=True).run() for seed in range(20))
