"""Fault-tolerant data parallelism: the training-side protocol on top of :mod:`.ftccl`.

Protocol of the reference trainer with ``transport: "ftccl"`` (reference: ``src/main.cpp:266-320, 350-478,
2955-2984, 3672-3767``):

* *collective phase gate* before every reduction: if peers wait to be admitted, or the world is smaller than it
  should be, update the topology (admits joiners, drops the dead);
* *shared state* = every parameter and optimizer tensor, with revision = training step; after a topology change
  everybody synchronises it (joiners receive it — this is how a restarted rank catches up without a checkpoint);
* gradients are all-reduced with retry; if too few peers remain the step is *dropped*: no optimizer update, the
  loss slot is discarded, state is re-synchronised at the old revision;
* after a committed step the revision is incremented.

Here a topology change also re-creates the process group of the new epoch and, for the ``fused`` reduction,
re-allocates the peer-memory windows and re-points the parameter / gradient buckets at them.  Failures are noticed
on the host (heartbeats at the master, exceptions from collectives) *between* steps; device-side waits are bounded.
When the world is smaller than ``expected_world`` the summed gradient is scaled by ``expected / actual`` so the
update keeps the magnitude of the full-batch mean.
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch
import torch.distributed as dist

from ..utils.logging import LOG
from ..utils.nvtx import gputx_range
from .dp import DataParallel
from .ftccl import FtPeer, Result, SharedStateSyncStrategy, TensorInfo


class FusedStepSnapshot:
    """Everything a fused reduce + optimizer step may change, captured before it runs, so that a step in which a
    peer stopped answering can be undone as a whole.

    The fused step is one kernel per bucket: buckets whose entry barrier passed before the peer fell silent have
    advanced their slice of m / v / master and stored new parameters into every member's window, later buckets have
    not, and the step counters are one ahead.  Dropping such a step must leave no trace (the reference's drop path
    re-synchronises state "at the old revision": ``src/main.cpp:3672-3713``), otherwise the half-applied slices
    would spread in the next shared-state synchronisation and the bias correction would run one step ahead.  The
    snapshot holds this member's slice of the sharded AdamW tensors, the Muon momentum / master tensors, the full
    parameter buckets (peers write into them) and the step counters; buffers are allocated once and reused."""

    def __init__(self):
        self._buffers = {}
        self._counters = []

    def _keep(self, key, t: torch.Tensor) -> None:
        buf = self._buffers.get(key)
        if buf is None or buf.shape != t.shape or buf.dtype != t.dtype or buf.device != t.device:
            buf = torch.empty_like(t)
            self._buffers[key] = buf
        buf.copy_(t)
        self._live.append((t, buf))

    @staticmethod
    def _optimizers(trainer):
        for opt in trainer.optimizers.values():
            yield opt
            for sub in ("adam", "muon"):
                if hasattr(opt, sub):
                    yield getattr(opt, sub)

    def capture(self, trainer, rank: int, world: int) -> None:
        self._live = []
        self._counters = [(opt, opt.step_count) for opt in self._optimizers(trainer)]
        for g in trainer.all_groups():
            self._keep(("param", g.name), g.data)
        for opt in self._optimizers(trainer):
            groups = getattr(opt, "groups", None)
            if groups is not None and getattr(opt, "flat_state", None) is not None:      # flat (shardable) AdamW
                for g, fs in zip(groups, opt.flat_state):
                    per = g.numel // world
                    for key, t in fs.items():
                        self._keep(("flat", id(opt), g.name, key), t[rank * per:(rank + 1) * per])
            elif isinstance(getattr(opt, "state", None), dict) and hasattr(opt, "named_params"):
                for name, _ in opt.named_params:
                    for key, t in opt.state.get(name, {}).items():
                        if torch.is_tensor(t):
                            self._keep(("state", id(opt), name, key), t)

    def restore(self) -> None:
        for t, buf in self._live:
            t.copy_(buf)
        for opt, count in self._counters:
            opt.step_count = count
        self._live = []


class FaultTolerantDataParallel:
    def __init__(self, peer: FtPeer, expected_world: int, min_world: int = 1, mode: str = "allreduce",
                 wait_for_full_world: bool = False, full_world_poll_s: float = 1.0):
        if mode not in ("allreduce", "fused"):
            raise ValueError("mode must be allreduce or fused")
        self.peer, self.expected_world, self.min_world, self.mode = peer, expected_world, min_world, mode
        self.wait_for_full_world = wait_for_full_world
        self.full_world_poll_s = full_world_poll_s
        self.gate_timeout_s = 30.0            # how long members wait for each other at the host-side step barrier
        self.inner: Optional[DataParallel] = None
        self.events: List[dict] = []          # topology changes with timestamps (recovery-time accounting)
        self.tx_bytes = self.rx_bytes = 0
        self.dropped_steps = 0
        self.ready_gate = None                # optional callable run right before a late joiner connects
        self._snapshot: Optional[FusedStepSnapshot] = None

    # the trainer reads these
    @property
    def rank(self) -> int:
        return self.peer.rank

    @property
    def world_size(self) -> int:
        # batch arithmetic (total_batch / micro / world) is defined by the nominal world
        return self.expected_world

    # ------------------------------------------------------------------------------------------
    def _shared_state(self, trainer) -> List[TensorInfo]:
        infos = [TensorInfo("group/" + g.name, g.data) for g in trainer.all_groups()]
        for opt in trainer.optimizers.values():
            for name, t in sorted(opt.state_tensors().items()):
                if name.endswith("__optimizer/step"):
                    continue
                infos.append(TensorInfo(name, t))
        if getattr(trainer, "data_state", None) is not None:
            # where the group's dataset iterator stands: travels with the rest to whoever receives the state, but a
            # difference in it alone is no reason for a transfer
            infos.append(TensorInfo("data/iterator_state", trainer.data_state, allow_content_inequality=True))
        return infos

    def _sync_state(self, trainer, joining: bool = False) -> bool:
        strategy = SharedStateSyncStrategy.RECEIVE_ONLY if joining else SharedStateSyncStrategy.ENFORCE_POPULAR
        with gputx_range("fbamtrain::ccl_state_broadcast"):
            res, info = self.peer.synchronize_shared_state(trainer.step_count, self._shared_state(trainer), strategy)
        if res != Result.SUCCESS:
            return False
        self.tx_bytes += info.tx_bytes
        self.rx_bytes += info.rx_bytes
        if info.revision != trainer.step_count:
            LOG("INFO", f"ftccl: adopting shared-state revision {info.revision} (was {trainer.step_count})")
            trainer.step_count = info.revision
            for opt in trainer.optimizers.values():
                opt.set_step(info.revision)
        return True     # fp32 master copies are optimizer tensors and were synchronised with the rest

    def _retopologize(self, trainer, joining: bool = False) -> bool:
        t0 = time.perf_counter()
        for _ in range(50):
            res = self.peer.update_topology(min_world=self.min_world)
            if res == Result.SUCCESS:
                break
            time.sleep(0.1)       # the reference retries every 100 ms on UpdateTopologyFailed
        else:
            return False
        if self.mode == "fused":
            old = None
            if self.inner is None:
                self.inner = DataParallel(mode="fused", group=None, window_transport="ipc")
                self.inner.attach_windows_only(trainer)
            else:
                old = (self.inner.rank, self.inner.world_size)
                old_owners = {id(opt.muon): dict(self.inner._muon_owner_map(opt.muon))
                              for opt in trainer.optimizers.values() if hasattr(opt, "muon") and old[1] > 1}
                self.inner.rebuild(trainer, None)
                self._old_muon_owners = old_owners
            self._recover_sharded_state(trainer, old)
        ok = self._sync_state(trainer, joining)
        self.events.append({"epoch": self.peer.epoch, "world": self.peer.world_size, "step": trainer.step_count,
                            "seconds": time.perf_counter() - t0})
        return ok

    def _recover_sharded_state(self, trainer, old) -> None:
        """The fused step keeps AdamW moments and fp32 masters current only in each member's slice of a bucket, and
        the slices move when the world changes: collect them from the members that are still here before the state
        is compared and handed to joiners.  Slices of members that are gone restart their moments from zero and
        take their masters from the (replicated) parameters; Muon momentum of matrices whose owner is gone restarts
        from zero as well."""
        from .dp import recover_sharded_state
        pairs = []
        for opt in self.inner._adamw_optimizers(trainer):
            for g, fs in zip(opt.groups, opt.flat_state):
                pairs.append((fs["m"], None))
                pairs.append((fs["v"], None))
                if "master" in fs:
                    pairs.append((fs["master"], g.data))
        if pairs and self.peer.world_size > 1:
            lost = recover_sharded_state(pairs, old, None)
            if lost:
                LOG("WARN", f"ftccl: {lost} optimizer-state slice(s) had no surviving owner; their moments restart")
        # Muon: the momentum of a matrix is current only on the rank that owned it in the old world (a world of
        # one owned everything); one summed exchange moves every matrix to where it is needed next
        old_owners = getattr(self, "_old_muon_owners", {}) or {}
        self._old_muon_owners = {}
        if self.peer.world_size > 1:
            bufs = []
            for opt in trainer.optimizers.values():
                if not hasattr(opt, "muon") or not opt.muon.named_params:
                    continue
                owners = old_owners.get(id(opt.muon))
                for name, _ in opt.muon.named_params:
                    buf = opt.muon.state[name]["momentum"]
                    if not (old is not None and (owners is None or owners[name] == old[0])):
                        buf.zero_()
                    bufs.append(buf)
            if bufs:
                flat = torch.cat([b.reshape(-1) for b in bufs])
                dist.all_reduce(flat)
                offset = 0
                for b in bufs:
                    b.copy_(flat[offset:offset + b.numel()].view_as(b))
                    offset += b.numel()
        if pairs and self.peer.world_size <= 1 and old is not None and old[1] > 1:
            # alone now: everything outside the old slice is stale
            for t, fallback in pairs:
                per = t.numel() // old[1]
                lo, hi = old[0] * per, (old[0] + 1) * per
                keep = t[lo:hi].clone()
                if fallback is None:
                    t.zero_()
                else:
                    t.copy_(fallback.to(t.dtype))
                t[lo:hi] = keep

    def attach(self, trainer) -> None:
        if self.peer.uid is None:
            # a peer that joins a running group builds its model first and only then announces itself, so that
            # the members are not held at their phase gate while it initialises
            if self.ready_gate is not None:
                self.ready_gate()
            if self.peer.connect() != Result.SUCCESS:
                raise RuntimeError("ftccl: cannot reach the membership master")
        joining = trainer.step_count == 0 and self.peer.epoch == 0 and getattr(self, "late_joiner", False)
        if not self._retopologize(trainer, joining):
            raise RuntimeError("ftccl: could not join the training group")

    def arm(self) -> None:
        if self.inner is not None:
            self.inner.arm()

    # ------------------------------------------------------------------------------------------
    def reduce_and_step(self, trainer) -> bool:
        peer = self.peer
        # Collective phase gate (host side, between kernels).  The members meet at the master before every
        # collective: a peer that left after the previous step, fell silent or waits for admission is noticed here,
        # before anything is launched that would wait for it on the device, and the members enter the fused
        # kernels within a network round trip of each other, so the bounded device-side waits stay short.
        # After a topology change the members pass the gate again, now together with whoever was admitted: a member
        # that re-formed the group on its own schedule (it was alone, or noticed the newcomer first) must not enter
        # the collective while the others still expect it at the gate.
        for _ in range(8):
            aligned = peer.gate(trainer.step_count, timeout_s=self.gate_timeout_s) if peer.world_size > 1 \
                else (peer.refresh_view() or not peer.membership_changed())
            changed = not aligned or peer.membership_changed() or peer.are_peers_pending()
            if changed and not self._retopologize(trainer):
                return self._drop(trainer, "topology update failed")
            while self.wait_for_full_world and peer.world_size < self.expected_world:
                time.sleep(self.full_world_poll_s)   # "not ready": the reference sleeps 1 s per round
                if peer.are_peers_pending():
                    changed = True
                    if not self._retopologize(trainer):
                        return self._drop(trainer, "topology update failed")
            if not changed:
                break
        else:
            return self._drop(trainer, "membership did not settle")
        if peer.world_size < self.min_world:
            return self._drop(trainer, "too few peers")
        scale = self.expected_world / max(1, peer.world_size)
        if self.mode == "fused" and peer.world_size > 1:
            self.inner.grad_scale = scale
            if self._snapshot is None:
                self._snapshot = FusedStepSnapshot()
            self._snapshot.capture(trainer, self.inner.rank, self.inner.world_size)
            self.inner.reduce_and_step(trainer)
            if not self._fused_step_completed(trainer):
                # a peer stopped answering inside the step: its bounded waits ran out and the kernels returned.
                # Some buckets were updated and some were not: undo all of it before anyone compares state.
                self._snapshot.restore()
                self._retopologize(trainer)
                return self._drop(trainer, "a device-side wait for a peer timed out")
        else:
            grads = [g.grad for g in trainer.all_groups()]
            if peer.world_size > 1:
                epoch_before, t0 = peer.epoch, time.perf_counter()
                with gputx_range("fbamtrain::ftccl_action_model_grad_allreduce"):
                    res, info = peer.all_reduce_multiple_with_retry(grads, [(trainer.step_count << 8) | k
                                                                            for k in range(len(grads))],
                                                                    min_world=self.min_world)
                self.tx_bytes += info.tx_bytes
                self.rx_bytes += info.rx_bytes
                if peer.epoch != epoch_before:    # a peer fell out during the collective; the retry re-formed the group
                    self.events.append({"epoch": peer.epoch, "world": peer.world_size, "step": trainer.step_count,
                                        "seconds": time.perf_counter() - t0})
                if res != Result.SUCCESS:
                    return self._drop(trainer, res.name)
                scale = self.expected_world / max(1, peer.world_size)
            if scale != 1.0:
                for g in grads:
                    g.mul_(scale)
            trainer.optimizers["action_model"].step()
            trainer.optimizers["frame_head"].step()
        return True

    def _fused_step_completed(self, trainer) -> bool:
        """Host-synchronises and reads the word the fused kernels set when a bounded wait expires."""
        from ..ops import native as nv
        torch.cuda.synchronize(trainer.device)
        word = nv.status_word(trainer.device)
        code = int(word.item())
        if code != 0:
            word.zero_()
            LOG("WARN", f"ftccl: fused step reported status {code}")
            return False
        return True

    def _drop(self, trainer, why: str) -> bool:
        """No update for this step; peers re-synchronise at the old revision."""
        LOG("WARN", f"ftccl: dropping step {trainer.step_count}: {why}")
        self.dropped_steps += 1
        if self.peer.world_size > 1:
            self._sync_state(trainer)
        return False

    def gather_optimizer_state(self, trainer) -> None:
        if self.inner is not None:
            self.inner.gather_optimizer_state(trainer)
