"""Dynamic membership for data parallelism over pipelines: whole pipelines join and leave a running job.

The reference combines ``ddp_parallel`` (transport ``ftccl``) with ``frame_head_parallel``: the recurrence master of
each pipeline is the fault-tolerant peer; after the gradient exchange it broadcasts a one-word commit / drop decision
to its frame workers, and after a dropped step or a topology change the state is broadcast again
(``src/main.cpp:549-586, 2563-2588, 3661-3711``).  Here:

* every pipeline is a job of its own with a static ``torch.distributed`` default group (stage-to-stage transfers,
  tensor parallelism); pipelines do not share a launcher, so one can be started or stopped without the others;
* the *leader* (rank 0 of the pipeline) is the only :class:`~.ftccl.FtPeer`: it heartbeats, meets the other leaders at
  the host-side step gate and votes for topology updates.  Membership is therefore per pipeline: a pipeline is
  admitted or dropped as a whole;
* after a topology round the leader broadcasts the outcome (epoch, number of pipelines, this pipeline's index, the
  address of the epoch's bootstrap store) over the static group, and every rank builds a :class:`~.ftccl.ScopedGroup`
  with the ranks in its own position of the other pipelines; parameters and optimizer state of the position are made
  equal there (a joining pipeline receives them; revision = training step);
* per step: gate → (topology update if the membership changed) → gradients summed over the position's group →
  one word per rank ("my exchange succeeded") reduced with MIN over the static group: the pipeline commits the step
  only if every position's exchange succeeded.  A failed exchange fails on every member of that position's group,
  so all pipelines take the same decision.  With fewer pipelines than expected the summed gradient is scaled by
  ``expected / actual``.

Failures are noticed on the host: a leader that stops heartbeating is evicted by the master, the others learn of it
at the next gate, before they launch a collective that would wait for it.
"""
from __future__ import annotations

import ipaddress
import time
from typing import List, Optional

import torch
import torch.distributed as dist

from ..utils.logging import LOG
from .ftccl import (FtPeer, Result, ScopedGroup, SharedStateSyncStrategy, TensorInfo, synchronize_shared_state)

_CONTROL_WORDS = 8


class FaultTolerantPipelineReplicas:
    def __init__(self, master_ip: str, master_port: int, device: torch.device, expected_replicas: int,
                 min_replicas: int = 1, late_joiner: bool = False, heartbeat_interval_s: float = 0.25,
                 collective_timeout_s: float = 30.0, gate_timeout_s: float = 30.0, stall_timeout_s: float = 300.0):
        """``stall_timeout_s``: when the leader has not reached its step gate for this long (it waits in a collective
        of the pipeline's own process group because another rank of the pipeline is gone), it stops heartbeating, so
        that the other pipelines drop this one instead of waiting for it at every gate (0 = never)."""
        if not dist.is_initialized():
            raise RuntimeError("the pipeline's own process group must be initialised first")
        self.device = device
        self.expected_replicas, self.min_replicas = expected_replicas, min_replicas
        self.late_joiner = late_joiner
        self.collective_timeout_s, self.gate_timeout_s = collective_timeout_s, gate_timeout_s
        self.position = dist.get_rank()                    # this rank's place inside its pipeline
        self.is_leader = self.position == 0
        self.peer: Optional[FtPeer] = None
        if self.is_leader:
            self.peer = FtPeer(master_ip, master_port, device, heartbeat_interval_s=heartbeat_interval_s,
                               collective_timeout_s=collective_timeout_s, owns_default_group=False,
                               progress_deadline_s=stall_timeout_s)
        self.group: Optional[ScopedGroup] = None
        self.epoch = 0
        self.replicas = 0                  # pipelines in the current topology
        self.replica_index = 0             # this pipeline's index among them
        self.events: List[dict] = []
        self.dropped_steps = 0
        self.tx_bytes = self.rx_bytes = 0

    # -- the leader's word to its pipeline ---------------------------------------------------------------------
    def _control(self, words: Optional[List[int]]) -> List[int]:
        """Broadcast of a few integers from the leader over the pipeline's static group."""
        t = torch.zeros(_CONTROL_WORDS, dtype=torch.int64, device=self.device)
        if self.is_leader:
            t[:len(words)] = torch.tensor(words, dtype=torch.int64)
        dist.broadcast(t, src=0)
        return [int(v) for v in t.tolist()]

    def _all_agree(self, ok: bool) -> bool:
        """One word per rank, MIN over the pipeline: the commit / drop decision."""
        t = torch.tensor([1 if ok else 0], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(int(t.item()))

    # -- topology ----------------------------------------------------------------------------------------------
    def _shared_state(self, trainer) -> List[TensorInfo]:
        infos = [TensorInfo("param/" + name, p.data) for name, p in trainer.named]
        for name, t in sorted(trainer.optimizer.state_tensors().items()):
            if not name.endswith("__optimizer/step"):
                infos.append(TensorInfo(name, t))
        if getattr(trainer, "data_state", None) is not None:
            # where the job's dataset iterator stands: travels with the rest to a pipeline that receives the state,
            # but a difference in it alone is no reason for a transfer
            infos.append(TensorInfo("data/iterator_state", trainer.data_state, allow_content_inequality=True))
        return infos

    def _retopologize(self, trainer, joining: bool = False) -> bool:
        t0 = time.perf_counter()
        words = None
        if self.is_leader:
            res = None
            for _ in range(50):
                self.peer.note_progress()              # waiting for the others' votes is not a stall of this pipeline
                res = self.peer.vote_topology(min_world=self.min_replicas)
                if res is not None:
                    break
                time.sleep(0.1)
            if res is None:
                words = [0]
            else:
                words = [1, int(res["epoch"]), int(res["world"]), int(res["ranks"][str(self.peer.uid)]),
                         int(ipaddress.IPv4Address(res["store"]["ip"])), int(res["store"]["port"])]
        ok, epoch, world, index, ip, port = self._control(words)[:6]
        if self.group is not None:
            self.group.close()
            self.group = None
        if not ok:
            return False
        self.epoch, self.replicas, self.replica_index = epoch, world, index
        synced = True
        if world > 1:
            try:
                self.group = ScopedGroup(str(ipaddress.IPv4Address(ip)), port, host_store=(index == 0 and self.is_leader),
                                         prefix=f"ftpipe/{epoch}/{self.position}", rank=index, world_size=world,
                                         device=self.device, timeout_s=self.collective_timeout_s)
                synced = self._sync_state(trainer, joining)
            except Exception as ex:  # noqa: BLE001
                LOG("WARN", f"ftccl: position {self.position} could not form its group for epoch {epoch}: {ex}")
                synced = False
        synced = self._all_agree(synced)
        self.events.append({"epoch": epoch, "replicas": world, "step": trainer.step_count,
                            "seconds": time.perf_counter() - t0})
        return synced

    def _sync_state(self, trainer, joining: bool = False) -> bool:
        strategy = SharedStateSyncStrategy.RECEIVE_ONLY if joining else SharedStateSyncStrategy.ENFORCE_POPULAR
        res, info = synchronize_shared_state(self.group, trainer.step_count, self._shared_state(trainer), strategy)
        if res != Result.SUCCESS:
            return False
        self.tx_bytes += info.tx_bytes
        self.rx_bytes += info.rx_bytes
        if info.revision != trainer.step_count:
            LOG("INFO", f"ftccl: adopting shared-state revision {info.revision} (was {trainer.step_count})")
            trainer.step_count = info.revision
            trainer.optimizer.set_step(info.revision)
        return True

    def attach(self, trainer) -> None:
        """Announces the pipeline to the master (the model is built by now, so the members are not held at their
        gate while it initialises) and joins the current topology."""
        if self.is_leader and self.peer.connect() != Result.SUCCESS:
            raise RuntimeError("ftccl: cannot reach the membership master")
        if not self._retopologize(trainer, joining=self.late_joiner):
            raise RuntimeError("ftccl: could not join the training group")

    # -- per step ----------------------------------------------------------------------------------------------
    def reduce(self, trainer, extra: Optional[torch.Tensor] = None) -> bool:
        """Sums the gradients of ``trainer.named`` (and ``extra``, e.g. the loss share) over the pipelines.  True:
        commit the step.  False: drop it (no optimizer update)."""
        for _ in range(8):
            words = None
            if self.is_leader:
                peer = self.peer
                peer.note_progress()
                if peer.world_size > 1:
                    aligned = peer.gate(trainer.step_count, timeout_s=self.gate_timeout_s)
                else:
                    peer.refresh_view()
                    aligned = not peer.membership_changed()
                words = [int(not aligned or peer.membership_changed() or peer.are_peers_pending())]
            changed = self._control(words)[0]
            if not changed:
                break
            if not self._retopologize(trainer):
                return self._drop(trainer, "topology update failed")
        else:
            return self._drop(trainer, "membership did not settle")
        if self.replicas < self.min_replicas:
            return self._drop(trainer, "too few pipelines")
        ok = True
        grads = [p.grad for _, p in trainer.named if p.grad is not None]
        if extra is not None:
            grads.append(extra)
        if self.replicas > 1:
            try:
                for g in grads:
                    self.group.all_reduce(g)
                    self.tx_bytes += g.numel() * g.element_size()
                if self.device.type == "cuda":
                    torch.cuda.synchronize(self.device)
            except Exception as ex:  # noqa: BLE001
                LOG("WARN", f"ftccl: gradient exchange of position {self.position} failed: {ex}")
                ok = False
        if not self._all_agree(ok):
            return self._drop(trainer, "a position's gradient exchange failed")
        scale = self.expected_replicas / max(1, self.replicas)
        if scale != 1.0:
            for g in grads:
                g.mul_(scale)
        return True

    def _drop(self, trainer, why: str) -> bool:
        LOG("WARN", f"ftccl: pipeline drops step {trainer.step_count}: {why}")
        self.dropped_steps += 1
        return False

    def leave(self) -> None:
        """Orderly departure between steps (all ranks of the pipeline call it)."""
        if self.group is not None:
            self.group.close()
            self.group = None
        if self.peer is not None:
            self.peer.leave()

    def inject_failure(self) -> None:
        """Host-side fault injection: the pipeline falls silent without telling the master."""
        if self.peer is not None:
            self.peer.inject_failure()
