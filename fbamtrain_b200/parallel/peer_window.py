"""Peer-memory windows: buffers that every rank of a group can load from and store to directly.

A ``PeerWindow`` owns one symmetric allocation per rank (same size everywhere), the table of all
ranks' device pointers to it, an optional NVSwitch multicast address, and is created collectively.
``PeerGroup`` bundles the windows of one communicator with the flag words and the epoch counter the
fused kernels synchronise on, and ``rebuild()`` re-creates everything after a membership change
(new group → new allocations → new pointer tables; epochs keep counting so stale flags can never
satisfy a wait).

The allocation and handle exchange is ``torch.distributed``'s symmetric-memory facility (CUDA VMM /
fabric handles exchanged through the group's store).  ``LocalPeerGroup`` lays the same interface
over plain buffers of ONE device, so that a single process can play several ranks in turn — used to
test the kernels' arithmetic without a second GPU (cross-rank waits are switched off there, because
kernels that wait on one another must never be separate launches on one device).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

MAX_RANKS = 8
FLAG_SLOTS = 16


def _ptr_array(ptrs: List[int]):
    arr = (C.c_void_p * MAX_RANKS)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class PeerWindow:
    """One symmetric buffer.  ``local`` is this rank's tensor; ``ptrs[r]`` is rank r's buffer as seen from here."""

    def __init__(self, local: torch.Tensor, ptrs: List[int], multicast_ptr: int = 0):
        self.local = local
        self.ptrs = ptrs
        self.multicast_ptr = multicast_ptr
        self.c_ptrs = _ptr_array(ptrs)

    def offset_ptrs(self, byte_offset: int):
        return _ptr_array([p + byte_offset for p in self.ptrs])


class _EpochCounter:
    """The flag-epoch bookkeeping shared by the window groups (``group``, ``device`` and ``epoch`` are the
    subclass's attributes)."""

    def _agree_on_epoch(self) -> None:
        """Every member continues from the highest epoch any member has used: the flag words of a new window start
        at zero, a long-running member's counter does not, and a wait compares the two."""
        t = torch.tensor([self.epoch], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        self.epoch = int(t.item())

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


class PeerGroup(_EpochCounter):
    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, use_multicast: bool = False):
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        if self.world_size > MAX_RANKS:
            raise ValueError(f"peer windows support at most {MAX_RANKS} ranks per group")
        self.use_multicast = use_multicast
        self.epoch = 0
        self.windows: Dict[str, PeerWindow] = {}
        self._build_flags()

    def _group_name(self) -> str:
        pg = self.group if self.group is not None else dist.group.WORLD
        return pg.group_name

    def allocate(self, name: str, numel: int, dtype: torch.dtype) -> PeerWindow:
        import torch.distributed._symmetric_memory as symm
        t = symm.empty(numel, dtype=dtype, device=self.device)
        t.zero_()
        handle = symm.rendezvous(t, self._group_name())
        ptrs = [int(p) for p in handle.buffer_ptrs]
        mc = int(handle.multicast_ptr) if (self.use_multicast and handle.multicast_ptr) else 0
        win = PeerWindow(t, ptrs, mc)
        win.handle = handle
        self.windows[name] = win
        return win

    def _build_flags(self) -> None:
        self.flags = self.allocate("__flags__", FLAG_SLOTS * MAX_RANKS, torch.int32)
        self.arrive = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._agree_on_epoch()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def rebuild(self, group: Optional[dist.ProcessGroup]) -> None:
        """Drops every window and re-creates the flag words for a new group; callers re-allocate their
        buffers (and re-point parameter / gradient views) afterwards.  The epoch counter is kept."""
        self.windows.clear()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self._build_flags()


class _RawDeviceBytes:
    """Exposes a raw device allocation through the CUDA array interface so that torch can wrap it without copying."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 2}


class IpcPeerGroup(_EpochCounter):
    """Same interface as :class:`PeerGroup`, with windows shared through CUDA IPC handles that the ranks exchange
    over the process group.  Nothing here depends on how long a process has been running, so a freshly started
    process can build windows together with long-running ones — which the fault-tolerant data-parallel mode needs
    after every membership change.  No NVSwitch multicast is bound to these windows (a departing rank must not
    leave a multicast binding behind); the fused kernels use plain peer loads and stores on them."""

    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, use_multicast: bool = False):
        if use_multicast:
            raise ValueError("IPC peer windows have no multicast address")
        self.group, self.device = group, device
        self.rank, self.world_size = dist.get_rank(group), dist.get_world_size(group)
        if self.world_size > MAX_RANKS:
            raise ValueError(f"peer windows support at most {MAX_RANKS} ranks per group")
        self.use_multicast = False
        self.epoch = 0
        self.windows: Dict[str, PeerWindow] = {}
        self._own: List[int] = []          # device allocations made for the current windows
        self._opened: List[int] = []       # peers' allocations opened for the current windows
        self._retired: List[int] = []      # own allocations of the previous group (local views may still be read)
        self._to_free: List[int] = []      # own allocations of the group before that, freed after the next barrier
        self._build_flags()

    def allocate(self, name: str, numel: int, dtype: torch.dtype) -> PeerWindow:
        from ..ops import native as nv
        lib = nv.lib()
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        nbytes = (nbytes + 255) // 256 * 256
        with torch.cuda.device(self.device):
            base = C.c_void_p()
            nv.check(lib.fbam_ipc_alloc(C.byref(base), C.c_longlong(nbytes)), "fbam_ipc_alloc")
            handle = (C.c_ubyte * 64)()
            nv.check(lib.fbam_ipc_export(base, handle), "fbam_ipc_export")
            everyone: List[Optional[bytes]] = [None] * self.world_size
            dist.all_gather_object(everyone, bytes(handle), group=self.group)
            ptrs = []
            for r, h in enumerate(everyone):
                if r == self.rank:
                    ptrs.append(int(base.value))
                    continue
                opened = C.c_void_p()
                nv.check(lib.fbam_ipc_open((C.c_ubyte * 64).from_buffer_copy(h), C.byref(opened)), "fbam_ipc_open")
                ptrs.append(int(opened.value))
                self._opened.append(int(opened.value))
        self._own.append(int(base.value))
        raw = torch.as_tensor(_RawDeviceBytes(int(base.value), nbytes), device=self.device)
        local = raw[:numel * torch.empty((), dtype=dtype).element_size()].view(dtype)
        win = PeerWindow(local, ptrs, 0)
        self.windows[name] = win
        return win

    def _build_flags(self) -> None:
        self.flags = self.allocate("__flags__", FLAG_SLOTS * MAX_RANKS, torch.int32)
        self.arrive = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._agree_on_epoch()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._free_retired()

    def _free_retired(self) -> None:
        """Frees the windows of the group before the previous one: every process that had them open has closed them
        at least one membership change ago, and no local tensor views them any more."""
        from ..ops import native as nv
        for address in self._to_free:
            nv.lib().fbam_ipc_free(C.c_void_p(address))
        self._to_free = []

    def release(self) -> None:
        """Closes the peers' windows (before leaving the group, or before re-building for a new one)."""
        from ..ops import native as nv
        torch.cuda.synchronize(self.device)
        for address in self._opened:
            nv.lib().fbam_ipc_close(C.c_void_p(address))
        self._opened = []
        self._to_free += self._retired
        self._retired = self._own
        self._own = []
        self.windows.clear()

    def rebuild(self, group: Optional[dist.ProcessGroup]) -> None:
        """New group, new allocations, new pointer tables; the epoch counter keeps counting.  Tensors that view the
        old windows stay readable until the NEXT rebuild (their memory is freed then)."""
        self.release()
        self.group = group
        self.rank, self.world_size = dist.get_rank(group), dist.get_world_size(group)
        self._build_flags()


class LocalPeerGroup:
    """Several emulated ranks inside one process on one device (see the module docstring)."""

    def __init__(self, world_size: int, device: torch.device):
        self.world_size, self.device = world_size, device
        self.epoch = 0
        self.windows: Dict[str, List[PeerWindow]] = {}
        self.arrive = torch.zeros(4, dtype=torch.int32, device=device)

    def allocate(self, name: str, numel: int, dtype: torch.dtype) -> List[PeerWindow]:
        bufs = [torch.zeros(numel, dtype=dtype, device=self.device) for _ in range(self.world_size)]
        ptrs = [b.data_ptr() for b in bufs]
        wins = [PeerWindow(b, ptrs, 0) for b in bufs]
        self.windows[name] = wins
        return wins

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch
