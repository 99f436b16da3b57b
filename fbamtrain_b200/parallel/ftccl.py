"""Fault-tolerant collective layer with dynamic peer membership.

The reference wraps Prime Intellect's PCCL (reference: ``ftccl/include/ftccl.h:9-229``,
``ftccl/src/ftccl_pccl.cpp:15-560``): a *master* process tracks membership; peers connect, are admitted at
topology updates that all accepted peers vote for, keep a revisioned *shared state* (all parameters and
optimizer tensors) consistent by hash comparison — outdated or newly joined peers receive the popular
content — and all-reduce with retry, dropping the step when too few peers remain.  This module provides
the same surface on top of plain TCP (control plane) and ``torch.distributed`` (data plane):

* :class:`MembershipMaster` — the master: peers register, heartbeat, vote for topology updates; it admits
  pending peers, evicts silent ones, numbers the topology *epoch* and hands out ranks and the address of the
  epoch's bootstrap store.
* :class:`FtPeer` — a peer: ``connect``, ``update_topology`` (re-rendezvous: tears the process group of the
  old epoch down and initialises the new one), ``are_peers_pending``, ``optimize_topology`` (a no-op here:
  behind NVSwitch every peer is equidistant, so there is no ring order to probe), ``synchronize_shared_state``,
  ``all_reduce`` / ``all_reduce_multiple_with_retry`` and world-size attributes.

Failures are detected on the host — a missed heartbeat at the master, or an exception from a collective — and
every device-side wait in the fused kernels is bounded, so a lost peer costs a dropped step, never a hung GPU.
``FtPeer.on_topology_change`` callbacks let owners of peer-memory windows rebuild them for the new group.

A peer normally owns the process's default ``torch.distributed`` group (one group per epoch).  A process that
already has a static default group (the ranks of one pipeline) keeps it: its leader only votes
(:meth:`FtPeer.vote_topology`) and every rank builds a :class:`ScopedGroup` — a stand-alone communicator over the
epoch's bootstrap store — for its own position (``parallel/ft_pipeline.py``).
"""
from __future__ import annotations

import datetime
import hashlib
import json
import socket
import threading
import time
from dataclasses import dataclass
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..utils.logging import LOG


class Result(Enum):
    SUCCESS = 0
    TOO_FEW_PEERS = 1
    RANK_CONNECTION_LOST = 2
    UPDATE_TOPOLOGY_FAILED = 3
    MASTER_CONNECTION_FAILED = 4
    INVALID_USAGE = 5


class SharedStateSyncStrategy(Enum):
    ENFORCE_POPULAR = 0
    RECEIVE_ONLY = 1
    SEND_ONLY = 2


class Attribute(Enum):
    GLOBAL_WORLD_SIZE = 0
    PEER_GROUP_WORLD_SIZE = 1
    NUM_DISTINCT_PEER_GROUPS = 2
    LARGEST_PEER_GROUP_WORLD_SIZE = 3


class QuantizationAlgorithm(Enum):
    NONE = 0
    MIN_MAX = 1
    ZERO_POINT_SCALE = 2


@dataclass
class ReduceInfo:
    world_size: int = 0
    tx_bytes: int = 0
    rx_bytes: int = 0


@dataclass
class SharedStateSyncInfo:
    tx_bytes: int = 0
    rx_bytes: int = 0
    revision: int = 0


@dataclass
class TensorInfo:
    name: str
    tensor: torch.Tensor
    allow_content_inequality: bool = False


def _send_json(sock: socket.socket, obj) -> None:
    sock.sendall((json.dumps(obj) + "\n").encode("utf-8"))


class _LineReader:
    def __init__(self, sock: socket.socket):
        self.sock, self.buf = sock, b""

    def read(self):
        while b"\n" not in self.buf:
            chunk = self.sock.recv(65536)
            if not chunk:
                raise ConnectionError("connection closed")
            self.buf += chunk
        line, self.buf = self.buf.split(b"\n", 1)
        return json.loads(line.decode("utf-8"))


# =================================================================================================
# master
# =================================================================================================
@dataclass
class _PeerRecord:
    uid: int
    peer_group: int
    ip: str
    last_seen: float
    accepted: bool = False
    vote: Optional[dict] = None
    conn: Optional[socket.socket] = None
    gate_step: Optional[int] = None


class MembershipMaster:
    """Runs in a thread (``start()``) or blocks (``run()``).  ``interrupt()`` stops it."""

    def __init__(self, ip: str = "127.0.0.1", port: int = 0, heartbeat_timeout_s: float = 2.0):
        self.ip, self.heartbeat_timeout_s = ip, heartbeat_timeout_s
        self._srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._srv.bind((ip, port))
        self._srv.listen(64)
        self.port = self._srv.getsockname()[1]
        self._lock = threading.Condition()
        self._peers: Dict[int, _PeerRecord] = {}
        self._next_uid = 1
        self.epoch = 0
        self._stop = False
        self._threads: List[threading.Thread] = []
        self._round_result: Optional[dict] = None
        self._round_id = 0

    # -- lifecycle ----------------------------------------------------------------------------
    def start(self) -> "MembershipMaster":
        t = threading.Thread(target=self.run, name="ftccl-master", daemon=True)
        t.start()
        self._threads.append(t)
        return self

    def run(self) -> None:
        self._srv.settimeout(0.2)
        while not self._stop:
            try:
                conn, addr = self._srv.accept()
            except socket.timeout:
                self._reap()
                continue
            except OSError:
                break
            t = threading.Thread(target=self._serve, args=(conn, addr), daemon=True)
            t.start()
        try:
            self._srv.close()
        except OSError:
            pass

    def interrupt(self) -> None:
        self._stop = True
        with self._lock:
            self._lock.notify_all()

    def await_termination(self, timeout: float = 5.0) -> None:
        for t in self._threads:
            t.join(timeout)

    # -- membership ---------------------------------------------------------------------------
    def _alive(self, rec: _PeerRecord) -> bool:
        return time.monotonic() - rec.last_seen <= self.heartbeat_timeout_s

    def _reap(self) -> None:
        with self._lock:
            dead = [uid for uid, r in self._peers.items() if not self._alive(r)]
            for uid in dead:
                LOG("WARN", f"ftccl master: peer {uid} missed its heartbeats, evicting")
                del self._peers[uid]
            if dead:
                self._lock.notify_all()

    def snapshot(self) -> dict:
        with self._lock:
            return {"epoch": self.epoch,
                    "accepted": sorted(u for u, r in self._peers.items() if r.accepted),
                    "pending": sorted(u for u, r in self._peers.items() if not r.accepted)}

    def _try_complete_round(self) -> None:
        """With the lock held: if every live accepted peer (or, at start-up, every pending peer that voted)
        has voted, admit the pending voters, renumber and publish the new topology."""
        live = {u: r for u, r in self._peers.items() if self._alive(r)}
        accepted = [r for r in live.values() if r.accepted]
        voters = [r for r in live.values() if r.vote is not None]
        if not voters:
            return
        if accepted and any(r.vote is None for r in accepted):
            return
        members = sorted((r for r in live.values() if r.accepted or r.vote is not None), key=lambda r: r.uid)
        if any(r.vote is None for r in members):
            return
        min_world = max(r.vote.get("min_world", 1) for r in members)
        if len(members) < min_world:
            return    # keep waiting for more peers to join
        self.epoch += 1
        leader = members[0]
        result = {"epoch": self.epoch, "world": len(members),
                  "ranks": {str(r.uid): i for i, r in enumerate(members)},
                  "store": {"ip": leader.ip, "port": leader.vote["free_port"]},
                  "groups": {str(r.uid): r.peer_group for r in members}}
        for r in members:
            r.accepted, r.vote = True, None
        self._round_id += 1
        self._round_result = dict(result, round=self._round_id)
        self._lock.notify_all()

    def _serve(self, conn: socket.socket, addr) -> None:
        reader = _LineReader(conn)
        uid = None
        try:
            while not self._stop:
                msg = reader.read()
                op = msg.get("op")
                with self._lock:
                    if uid is not None and uid in self._peers:
                        self._peers[uid].last_seen = time.monotonic()
                if op == "connect":
                    with self._lock:
                        uid = self._next_uid
                        self._next_uid += 1
                        self._peers[uid] = _PeerRecord(uid, int(msg.get("peer_group", 0)), msg.get("ip", addr[0]),
                                                       time.monotonic(), conn=conn)
                        self._lock.notify_all()
                    _send_json(conn, {"ok": True, "uid": uid})
                elif op == "heartbeat":
                    with self._lock:
                        known = uid in self._peers
                        snap = {"epoch": self.epoch,
                                "pending": sum(1 for r in self._peers.values() if not r.accepted),
                                "world": sum(1 for r in self._peers.values() if r.accepted and self._alive(r))}
                    _send_json(conn, dict(snap, ok=known))
                elif op == "pending":
                    with self._lock:
                        n = sum(1 for r in self._peers.values() if not r.accepted and self._alive(r))
                    _send_json(conn, {"ok": True, "pending": n})
                elif op == "vote":
                    deadline = time.monotonic() + float(msg.get("timeout", 30.0))
                    with self._lock:
                        if uid not in self._peers:
                            _send_json(conn, {"ok": False, "error": "evicted"})
                            continue
                        start_round = self._round_id
                        self._peers[uid].vote = msg
                        self._try_complete_round()
                        while self._round_id == start_round and not self._stop:
                            remaining = deadline - time.monotonic()
                            if remaining <= 0:
                                break
                            self._lock.wait(min(0.2, remaining))
                            if uid in self._peers:
                                self._peers[uid].last_seen = time.monotonic()
                            # evict silent peers so that a dead accepted peer cannot block the round
                            for u in [u for u, r in self._peers.items() if not self._alive(r) and u != uid]:
                                del self._peers[u]
                            if self._round_id == start_round:
                                self._try_complete_round()
                        if self._round_id != start_round and str(uid) in self._round_result["ranks"]:
                            res = dict(self._round_result, ok=True)
                        else:
                            if uid in self._peers:
                                self._peers[uid].vote = None
                            res = {"ok": False, "error": "timeout"}
                    _send_json(conn, res)
                elif op == "gate":
                    # Step barrier on the host: answers once every live accepted peer has reached the same step's
                    # phase gate, or as soon as the membership differs from the caller's epoch (someone left, was
                    # evicted or waits for admission) — then the caller must update the topology first.
                    step = int(msg.get("step", -1))
                    deadline = time.monotonic() + float(msg.get("timeout", 30.0))
                    with self._lock:
                        if uid not in self._peers:
                            _send_json(conn, {"ok": False, "error": "evicted"})
                            continue
                        self._peers[uid].gate_step = step
                        self._lock.notify_all()
                        res = None
                        while not self._stop:
                            live = [r for r in self._peers.values() if self._alive(r) or r.uid == uid]
                            accepted = [r for r in live if r.accepted]
                            pending = [r for r in live if not r.accepted]
                            changed = pending or int(msg.get("epoch", self.epoch)) != self.epoch or \
                                len(accepted) != int(msg.get("world", len(accepted)))
                            if changed:
                                res = {"ok": True, "aligned": False, "world": len(accepted), "pending": len(pending),
                                       "epoch": self.epoch}
                                break
                            if all(getattr(r, "gate_step", None) is not None and r.gate_step >= step for r in accepted):
                                res = {"ok": True, "aligned": True, "world": len(accepted), "pending": 0,
                                       "epoch": self.epoch}
                                break
                            remaining = deadline - time.monotonic()
                            if remaining <= 0:
                                res = {"ok": True, "aligned": False, "world": len(accepted), "pending": 0,
                                       "epoch": self.epoch, "timeout": True}
                                break
                            self._lock.wait(min(0.05, remaining))
                            if uid not in self._peers:
                                res = {"ok": False, "error": "evicted"}
                                break
                            self._peers[uid].last_seen = time.monotonic()
                            for u in [u for u, r in self._peers.items() if not self._alive(r) and u != uid]:
                                del self._peers[u]
                        res = res or {"ok": False, "error": "stopped"}
                    _send_json(conn, res)
                elif op == "leave":
                    with self._lock:
                        self._peers.pop(uid, None)
                        self._lock.notify_all()
                    _send_json(conn, {"ok": True})
                    break
                else:
                    _send_json(conn, {"ok": False, "error": f"unknown op {op}"})
        except (ConnectionError, OSError, json.JSONDecodeError):
            pass
        finally:
            try:
                conn.close()
            except OSError:
                pass


class NativeMembershipMaster:
    """The same service implemented in the native runtime (``csrc/runtime/membership.cpp``): one accept thread and
    one thread per peer connection inside the library, no Python in the request path.  Drop-in for
    :class:`MembershipMaster` (``start`` / ``port`` / ``snapshot`` / ``interrupt`` / ``await_termination``)."""

    def __init__(self, ip: str = "127.0.0.1", port: int = 0, heartbeat_timeout_s: float = 2.0):
        self.ip, self._want_port, self.heartbeat_timeout_s = ip, port, heartbeat_timeout_s
        self.port = 0
        self._handle = None

    def start(self) -> "NativeMembershipMaster":
        import ctypes as C
        from .. import runtime
        out = C.c_int(0)
        handle = runtime.lib().fbam_master_start(self.ip.encode(), self._want_port, self.heartbeat_timeout_s,
                                                 C.byref(out))
        if not handle:
            raise OSError(f"cannot start the membership master on {self.ip}:{self._want_port}")
        self._handle, self.port = handle, out.value
        return self

    def run(self) -> None:
        """Blocks until interrupted (for a stand-alone master process)."""
        if self._handle is None:
            self.start()
        while self._handle is not None:
            time.sleep(0.2)

    def snapshot(self) -> dict:
        import ctypes as C
        from .. import runtime
        buf = C.create_string_buffer(1 << 16)
        runtime.lib().fbam_master_snapshot(self._handle, buf, len(buf))
        return json.loads(buf.value.decode())

    def interrupt(self) -> None:
        if self._handle is not None:
            from .. import runtime
            handle, self._handle = self._handle, None
            runtime.lib().fbam_master_stop(handle)

    def await_termination(self, timeout: float = 5.0) -> None:
        return None


def create_master(ip: str = "127.0.0.1", port: int = 0, heartbeat_timeout_s: float = 2.0, native: Optional[bool] = None):
    """The membership master for a job: the native service when the runtime library is built (or ``native=True``),
    the Python one otherwise."""
    if native is None:
        from .. import runtime
        native = runtime.available()
    cls = NativeMembershipMaster if native else MembershipMaster
    return cls(ip, port, heartbeat_timeout_s)


# =================================================================================================
# peer
# =================================================================================================
def _free_port(ip: str) -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((ip, 0))
        return s.getsockname()[1]


def tensor_hash(t: torch.Tensor) -> str:
    return tensor_hashes([t])[0]


def tensor_hashes(tensors: Sequence[torch.Tensor]) -> List[str]:
    """Content fingerprints.  CUDA tensors are fingerprinted on the device (one kernel per tensor, one read-back
    for all of them); host tensors with BLAKE2b.  Peers only compare fingerprints of the same kind."""
    out: List[Optional[str]] = [None] * len(tensors)
    on_gpu = [i for i, t in enumerate(tensors) if t.is_cuda and t.numel()]
    if on_gpu:
        import ctypes as C
        from ..ops import native as nv
        dev = tensors[on_gpu[0]].device
        words = torch.zeros(len(on_gpu), 2, dtype=torch.int64, device=dev)
        keep = []
        for slot, i in enumerate(on_gpu):
            data = tensors[i].detach().contiguous()
            keep.append(data)
            nv.check(nv.lib().fbam_fingerprint(nv.ptr(data), C.c_longlong(data.numel() * data.element_size()),
                                               nv.ptr(words[slot]), nv.stream_ptr()), "fbam_fingerprint")
        host = words.cpu()
        for slot, i in enumerate(on_gpu):
            out[i] = f"{int(host[slot, 0]) & (2 ** 64 - 1):016x}{int(host[slot, 1]) & (2 ** 64 - 1):016x}"
    for i, t in enumerate(tensors):
        if out[i] is None:
            data = t.detach().contiguous().cpu()
            raw = data.view(torch.uint8).numpy().tobytes() if data.numel() else b""
            out[i] = hashlib.blake2b(raw, digest_size=16).hexdigest()
    return out


class _DefaultGroupComm:
    """The process's default ``torch.distributed`` group behind the small interface the shared-state exchange needs."""

    def __init__(self, rank: int, world_size: int):
        self.rank, self.world_size = rank, world_size

    def all_gather_object(self, obj) -> list:
        out: List[Optional[object]] = [None] * self.world_size
        dist.all_gather_object(out, obj)
        return out

    def broadcast(self, tensor: torch.Tensor, src: int) -> None:
        dist.broadcast(tensor, src=src)


class ScopedGroup:
    """A communicator of its own, next to whatever default group the process has: the members rendezvous through a
    TCP store at a known address (one member hosts it) under a prefix that names the group.  Gloo on CPU tensors,
    NCCL on CUDA tensors.  Used for the same-position ranks of pipelines that come and go
    (``parallel/ft_pipeline.py``); torn down and rebuilt at every topology epoch."""

    def __init__(self, store_ip: str, store_port: int, host_store: bool, prefix: str, rank: int, world_size: int,
                 device: torch.device, timeout_s: float = 30.0):
        self.rank, self.world_size, self.device = rank, world_size, device
        timeout = datetime.timedelta(seconds=timeout_s)
        self._store = dist.TCPStore(store_ip, store_port, None, host_store, timeout=timeout, wait_for_workers=False)
        scoped = dist.PrefixStore(prefix, self._store)
        if device.type == "cuda":
            self._pg = dist.ProcessGroupNCCL(scoped, rank, world_size, timeout)
        else:
            self._pg = dist.ProcessGroupGloo(scoped, rank, world_size, timeout=timeout)

    def all_reduce(self, tensor: torch.Tensor) -> None:
        self._pg.allreduce([tensor]).wait()

    def broadcast(self, tensor: torch.Tensor, src: int) -> None:
        opts = dist.BroadcastOptions()
        opts.rootRank, opts.rootTensor = src, 0
        self._pg.broadcast([tensor], opts).wait()

    def all_gather_object(self, obj) -> list:
        import pickle
        raw = pickle.dumps(obj)
        size = torch.tensor([len(raw)], dtype=torch.int64, device=self.device)
        sizes = [torch.zeros_like(size) for _ in range(self.world_size)]
        self._pg.allgather([sizes], [size]).wait()
        longest = max(int(t.item()) for t in sizes)
        mine = torch.zeros(longest, dtype=torch.uint8, device=self.device)
        mine[:len(raw)] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device)
        everyone = [torch.zeros_like(mine) for _ in range(self.world_size)]
        self._pg.allgather([everyone], [mine]).wait()
        return [pickle.loads(bytes(t[:int(n.item())].cpu().numpy().tobytes())) for t, n in zip(everyone, sizes)]

    def close(self) -> None:
        pg, self._pg = self._pg, None
        if pg is not None and hasattr(pg, "abort") and self.device.type == "cuda":
            try:
                pg.abort()          # do not wait for members that are gone
            except Exception:  # noqa: BLE001
                pass
        del pg
        self._store = None


def synchronize_shared_state(comm, revision: int, infos: Sequence[TensorInfo],
                             strategy: SharedStateSyncStrategy = SharedStateSyncStrategy.ENFORCE_POPULAR
                             ) -> Tuple[Result, SharedStateSyncInfo]:
    """Makes every member of ``comm`` (``rank``, ``world_size``, ``all_gather_object``, ``broadcast``) hold the same
    content for the named tensors.  Members exchange (revision, hash of all tensors); the donor is a member with the
    highest revision whose hash is the most common one at that revision (lowest rank on ties); every member whose
    hash differs receives the donor's tensors."""
    out = SharedStateSyncInfo(revision=revision)
    if comm.world_size <= 1:
        return Result.SUCCESS, out
    h = hashlib.blake2b(digest_size=16)
    compared = [ti for ti in infos if not ti.allow_content_inequality]
    for ti, digest in zip(compared, tensor_hashes([ti.tensor for ti in compared])):
        h.update(ti.name.encode())
        h.update(digest.encode())
    mine = (int(revision), h.hexdigest(), strategy.value)
    try:
        everyone = comm.all_gather_object(mine)
        candidates = [(r, rev, hh) for r, (rev, hh, st) in enumerate(everyone)
                      if st != SharedStateSyncStrategy.RECEIVE_ONLY.value]
        if not candidates:
            return Result.INVALID_USAGE, out
        top = max(rev for _, rev, _ in candidates)
        counts: Dict[str, int] = {}
        for _, rev, hh in candidates:
            if rev == top:
                counts[hh] = counts.get(hh, 0) + 1
        popular = max(counts.items(), key=lambda kv: (kv[1], ))[0]
        donor = min(r for r, rev, hh in candidates if rev == top and hh == popular)
        differs = [(rev, hh) != (top, popular) for (rev, hh, _) in everyone]
        out.revision = top
        if any(differs):
            for ti in infos:
                buf = ti.tensor if ti.tensor.is_contiguous() else ti.tensor.contiguous()
                comm.broadcast(buf, donor)
                if buf is not ti.tensor:
                    ti.tensor.copy_(buf)
                nbytes = buf.numel() * buf.element_size()
                if comm.rank == donor:
                    out.tx_bytes += nbytes * sum(differs)
                elif differs[comm.rank]:
                    out.rx_bytes += nbytes
    except Exception as ex:  # noqa: BLE001
        LOG("WARN", f"ftccl: shared-state synchronisation failed: {ex}")
        return Result.RANK_CONNECTION_LOST, out
    return Result.SUCCESS, out


class FtPeer:
    def __init__(self, master_ip: str, master_port: int, device: torch.device, peer_group: int = 0,
                 my_ip: str = "127.0.0.1", heartbeat_interval_s: float = 0.25, collective_timeout_s: float = 30.0,
                 p2p_connection_pool_size: int = 16, owns_default_group: bool = True,
                 progress_deadline_s: float = 0.0):
        """``owns_default_group=False``: the process has a default ``torch.distributed`` group of its own that this
        peer must leave alone (it then only connects, heartbeats, gates and votes; see :meth:`vote_topology`).

        ``progress_deadline_s`` > 0: the heartbeat thread vouches for the training thread only while that thread
        keeps calling :meth:`note_progress`; after this many seconds without a call the peer stops heartbeating and
        closes its connection, so the master evicts it like a process that died.  For peers whose training thread can
        block for a long time in something the master cannot see (the leader of a pipeline waits in a collective of
        its own process group when another rank of the pipeline has died)."""
        self.owns_default_group = owns_default_group
        self.progress_deadline_s = progress_deadline_s
        self._last_progress = time.monotonic()
        self.master_addr = (master_ip, master_port)
        self.device, self.peer_group, self.my_ip = device, peer_group, my_ip
        self.heartbeat_interval_s, self.collective_timeout_s = heartbeat_interval_s, collective_timeout_s
        self.p2p_connection_pool_size = p2p_connection_pool_size
        self.uid: Optional[int] = None
        self.epoch = 0
        self.rank = 0
        self.world_size = 0
        self._groups: Dict[str, int] = {}
        self._sock: Optional[socket.socket] = None
        self._reader: Optional[_LineReader] = None
        self._io = threading.Lock()
        self._hb_stop = threading.Event()
        self._hb_thread: Optional[threading.Thread] = None
        self._master_view = {"epoch": 0, "pending": 0, "world": 0, "ok": True}
        self.on_topology_change: List[Callable[["FtPeer"], None]] = []
        self.alive = True

    # -- control plane ------------------------------------------------------------------------
    def _rpc(self, msg: dict, timeout: float = 10.0) -> dict:
        with self._io:
            if self._sock is None:
                raise ConnectionError("not connected to the master")
            self._sock.settimeout(timeout)
            _send_json(self._sock, msg)
            return self._reader.read()

    def connect(self, retries: int = 50) -> Result:
        last = None
        for _ in range(retries):
            try:
                self._sock = socket.create_connection(self.master_addr, timeout=5.0)
                self._reader = _LineReader(self._sock)
                res = self._rpc({"op": "connect", "peer_group": self.peer_group, "ip": self.my_ip})
                self.uid = int(res["uid"])
                self._last_progress = time.monotonic()
                self._hb_stop.clear()
                self._hb_thread = threading.Thread(target=self._heartbeat_loop, name="ftccl-heartbeat", daemon=True)
                self._hb_thread.start()
                return Result.SUCCESS
            except OSError as ex:
                last = ex
                time.sleep(0.1)
        LOG("ERR", f"ftccl: cannot reach the master at {self.master_addr}: {last}")
        return Result.MASTER_CONNECTION_FAILED

    def note_progress(self) -> None:
        """The training thread is alive and moving (see ``progress_deadline_s``)."""
        self._last_progress = time.monotonic()

    def _heartbeat_loop(self) -> None:
        while not self._hb_stop.wait(self.heartbeat_interval_s):
            if self.progress_deadline_s > 0 and time.monotonic() - self._last_progress > self.progress_deadline_s:
                LOG("ERR", f"ftccl: no progress for {self.progress_deadline_s:.0f} s; this peer stops vouching for "
                           "its training thread and leaves the group")
                self._master_view = dict(self._master_view, ok=False)
                with self._io:
                    if self._sock is not None:
                        try:
                            self._sock.close()
                        except OSError:
                            pass
                        self._sock = None
                return
            try:
                self._master_view = self._rpc({"op": "heartbeat"}, timeout=5.0)
            except (OSError, ConnectionError, json.JSONDecodeError):
                self._master_view = dict(self._master_view, ok=False)
                return

    def refresh_view(self) -> None:
        """Asks the master for its current view NOW (the heartbeat thread's copy can be one interval old, which is
        longer than a training step on a fast device)."""
        try:
            self._master_view = self._rpc({"op": "heartbeat"}, timeout=5.0)
        except (OSError, ConnectionError, json.JSONDecodeError):
            self._master_view = dict(self._master_view, ok=False)

    def gate(self, step: int, timeout_s: float = 30.0) -> bool:
        """Host-side step barrier through the master.  True: every member of the current topology has reached the
        phase gate of ``step`` — launch the collective.  False: the membership differs from this peer's topology
        (or someone did not arrive in time) — update the topology before launching anything."""
        try:
            res = self._rpc({"op": "gate", "step": int(step), "epoch": self.epoch, "world": self.world_size,
                             "timeout": timeout_s}, timeout=timeout_s + 10.0)
        except (OSError, ConnectionError, json.JSONDecodeError):
            self._master_view = dict(self._master_view, ok=False)
            return False
        if not res.get("ok"):
            self._master_view = dict(self._master_view, ok=False)
            return False
        self._master_view = {"epoch": res.get("epoch", self.epoch), "pending": res.get("pending", 0),
                             "world": res.get("world", self.world_size), "ok": True}
        return bool(res.get("aligned"))

    def are_peers_pending(self) -> bool:
        try:
            return int(self._rpc({"op": "pending"})["pending"]) > 0
        except (OSError, ConnectionError):
            return False

    def membership_changed(self) -> bool:
        """Host-side check before launching collectives: True when the master's view differs from the
        topology this peer is running with (someone was evicted or waits to be admitted)."""
        v = self._master_view
        return (not v.get("ok", True)) or v.get("pending", 0) > 0 or (
            self.world_size > 0 and v.get("world", self.world_size) != self.world_size)

    def vote_topology(self, min_world: int = 1, timeout_s: float = 30.0) -> Optional[dict]:
        """Votes for a topology update and returns the master's answer once all accepted peers have voted (None when
        the round failed): ``epoch``, ``world``, ``ranks`` (uid → rank), ``groups`` (uid → peer group) and ``store``
        (address of the epoch's bootstrap store, a free port on the peer with rank 0).  Takes the new epoch, world
        size and rank but leaves process groups alone — :meth:`update_topology` builds the default group from the
        answer; a caller with its own communicators builds those."""
        try:
            res = self._rpc({"op": "vote", "free_port": _free_port(self.my_ip), "min_world": min_world,
                             "timeout": timeout_s}, timeout=timeout_s + 10.0)
        except (OSError, ConnectionError) as ex:
            LOG("ERR", f"ftccl: topology vote failed: {ex}")
            return None
        if not res.get("ok"):
            return None
        self.epoch = int(res["epoch"])
        self.world_size = int(res["world"])
        self.rank = int(res["ranks"][str(self.uid)])
        self._groups = res.get("groups", {})
        self._master_view = dict(self._master_view, world=self.world_size, pending=0, ok=True)
        return res

    def update_topology(self, min_world: int = 1, timeout_s: float = 30.0) -> Result:
        """Votes for a topology update and, once all accepted peers have voted, re-rendezvouses: the old
        process group is destroyed and the new epoch's group initialised with the ranks the master assigned."""
        if not self.owns_default_group:
            return Result.INVALID_USAGE
        res = self.vote_topology(min_world, timeout_s)
        if res is None:
            return Result.UPDATE_TOPOLOGY_FAILED
        self._teardown_group()
        store = res["store"]
        backend = "nccl" if self.device.type == "cuda" else "gloo"
        kwargs = {"device_id": self.device} if self.device.type == "cuda" else {}
        # Process-group names restart from "0" after destroy_process_group(); caches keyed by group name (the
        # symmetric-memory rendezvous among them) must not see an old epoch's group under a new epoch's name.
        import torch.distributed.distributed_c10d as c10d
        c10d._world.group_count = max(c10d._world.group_count, 64 * self.epoch)
        try:
            dist.init_process_group(backend, init_method=f"tcp://{store['ip']}:{store['port']}", rank=self.rank,
                                    world_size=self.world_size,
                                    timeout=datetime.timedelta(seconds=self.collective_timeout_s), **kwargs)
        except Exception as ex:  # noqa: BLE001
            LOG("ERR", f"ftccl: process-group initialisation for epoch {self.epoch} failed: {ex}")
            return Result.UPDATE_TOPOLOGY_FAILED
        self._master_view = dict(self._master_view, world=self.world_size, pending=0, ok=True)
        for cb in self.on_topology_change:
            cb(self)
        return Result.SUCCESS

    def optimize_topology(self) -> Result:
        """Ring-order optimisation by bandwidth probing has nothing to do behind an NVSwitch (every pair of
        GPUs has the same bandwidth); kept for API parity."""
        return Result.SUCCESS if self.world_size > 0 else Result.INVALID_USAGE

    def get_attribute(self, attr: Attribute) -> int:
        if attr == Attribute.GLOBAL_WORLD_SIZE:
            return self.world_size
        sizes: Dict[int, int] = {}
        for g in self._groups.values():
            sizes[g] = sizes.get(g, 0) + 1
        if attr == Attribute.PEER_GROUP_WORLD_SIZE:
            return sizes.get(self.peer_group, 0)
        if attr == Attribute.NUM_DISTINCT_PEER_GROUPS:
            return len(sizes)
        return max(sizes.values()) if sizes else 0

    def _teardown_group(self) -> None:
        if self.owns_default_group and dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass

    # -- data plane ---------------------------------------------------------------------------
    def all_reduce(self, tensor: torch.Tensor, tag: int = 0,
                   quantization: QuantizationAlgorithm = QuantizationAlgorithm.NONE) -> Tuple[Result, ReduceInfo]:
        """Sum all-reduce.  A failed collective (lost peer) returns RANK_CONNECTION_LOST and leaves
        ``tensor`` unspecified: callers retry after a topology update or drop the step."""
        info = ReduceInfo(world_size=self.world_size)
        if self.world_size <= 1:
            return (Result.TOO_FEW_PEERS if self.world_size < 1 else Result.SUCCESS), info
        if quantization != QuantizationAlgorithm.NONE:
            return self._all_reduce_quantized(tensor, tag, quantization, info)
        try:
            dist.all_reduce(tensor)
            if tensor.is_cuda:
                torch.cuda.synchronize(tensor.device)
        except Exception as ex:  # noqa: BLE001
            LOG("WARN", f"ftccl: all-reduce (tag {tag}) failed: {ex}")
            return Result.RANK_CONNECTION_LOST, info
        nbytes = tensor.numel() * tensor.element_size()
        info.tx_bytes = info.rx_bytes = 2 * nbytes * (self.world_size - 1) // self.world_size
        return Result.SUCCESS, info

    def _all_reduce_quantized(self, tensor: torch.Tensor, tag: int, quantization: QuantizationAlgorithm,
                              info: ReduceInfo) -> Tuple[Result, ReduceInfo]:
        """Lossy sum for slow links (the reference exposes PCCL's MinMax / ZeroPointScale options,
        ``ftccl/include/ftccl.h``): every peer sends its contribution as 8-bit codes with a per-tensor affine
        map, all peers decode and sum in fp32 in rank order — a quarter of the bytes of an fp32 exchange.
        MinMax maps [min, max] onto 0..255; ZeroPointScale uses a symmetric scale around zero (code 128 = 0)."""
        x = tensor.detach().float().reshape(-1)
        if quantization == QuantizationAlgorithm.MIN_MAX:
            lo, hi = x.min(), x.max()
        else:
            hi = x.abs().max()
            lo = -hi
        span = torch.clamp(hi - lo, min=1e-30)
        codes = torch.clamp(torch.round((x - lo) / span * 255.0), 0, 255).to(torch.uint8)
        meta = torch.stack([lo, span]).float()
        try:
            all_codes = [torch.empty_like(codes) for _ in range(self.world_size)]
            all_meta = [torch.empty_like(meta) for _ in range(self.world_size)]
            dist.all_gather(all_codes, codes)
            dist.all_gather(all_meta, meta)
            if tensor.is_cuda:
                torch.cuda.synchronize(tensor.device)
        except Exception as ex:  # noqa: BLE001
            LOG("WARN", f"ftccl: quantised all-reduce (tag {tag}) failed: {ex}")
            return Result.RANK_CONNECTION_LOST, info
        total = torch.zeros_like(x)
        for c, mt in zip(all_codes, all_meta):
            total += c.float() * (mt[1] / 255.0) + mt[0]
        tensor.copy_(total.view_as(tensor).to(tensor.dtype))
        info.tx_bytes = info.rx_bytes = (codes.numel() + 8) * (self.world_size - 1)
        return Result.SUCCESS, info

    def all_reduce_multiple_with_retry(self, tensors: Sequence[torch.Tensor], tags: Sequence[int],
                                       min_world: int = 2, max_in_flight: int = 8,
                                       max_retries: int = 3) -> Tuple[Result, ReduceInfo]:
        """All-reduces every tensor; on a lost connection restores the inputs, re-rendezvouses and retries.
        Returns TOO_FEW_PEERS when fewer than ``min_world`` peers remain (the caller drops the step)."""
        backups = [t.clone() for t in tensors]
        total = ReduceInfo(world_size=self.world_size)
        for attempt in range(max_retries + 1):
            if self.world_size < min_world:
                return Result.TOO_FEW_PEERS, total
            failed = False
            for t, tag in zip(tensors, tags):
                res, info = self.all_reduce(t, tag)
                if res != Result.SUCCESS:
                    failed = True
                    break
                total.tx_bytes += info.tx_bytes
                total.rx_bytes += info.rx_bytes
            if not failed:
                total.world_size = self.world_size
                return Result.SUCCESS, total
            for t, b in zip(tensors, backups):
                t.copy_(b)
            if self.update_topology(min_world=1) != Result.SUCCESS:
                return Result.UPDATE_TOPOLOGY_FAILED, total
        return Result.RANK_CONNECTION_LOST, total

    def synchronize_shared_state(self, revision: int, infos: Sequence[TensorInfo],
                                 strategy: SharedStateSyncStrategy = SharedStateSyncStrategy.ENFORCE_POPULAR
                                 ) -> Tuple[Result, SharedStateSyncInfo]:
        """:func:`synchronize_shared_state` over this peer's process group."""
        return synchronize_shared_state(_DefaultGroupComm(self.rank, self.world_size), revision, infos, strategy)

    # -- leaving / failure injection ----------------------------------------------------------
    def leave(self) -> None:
        """Orderly departure between steps."""
        self._hb_stop.set()
        try:
            self._rpc({"op": "leave"}, timeout=2.0)
        except (OSError, ConnectionError):
            pass
        self._close()

    def inject_failure(self) -> None:
        """Host-side fault injection: the peer falls silent (no heartbeats, sockets closed) without telling
        anyone, as a crashed process would.  The device context is untouched."""
        self._hb_stop.set()
        self._close()

    def _close(self) -> None:
        self.alive = False
        self._teardown_group()
        with self._io:
            if self._sock is not None:
                try:
                    self._sock.close()
                except OSError:
                    pass
                self._sock = None
