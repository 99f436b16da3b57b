"""Thin collective-communication layer over ``torch.distributed`` (NCCL on GPUs, gloo on CPU ranks).

It offers the operations of the reference's NCCL wrapper (reference: ``ccl/include/ccl.h:11-70``,
``ccl/src/ccl_nccl.cpp:67-378``): communicator creation from a rendezvous, subset communicators,
destroy with abort fallback, 256-byte string send/recv, a verified barrier (one-element all-reduce
whose result must equal the world size), asynchronous send / recv / broadcast of raw buffers,
sum all-reduce and all-gather.  "Async" calls return the ``Work`` handle; on NCCL they are ordered on
the current CUDA stream.  Errors carry the backend's message (the reference appends
``ncclCommGetAsyncError``).
"""
from __future__ import annotations

import datetime
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.distributed as dist

STRING_BYTES = 256


class CclError(RuntimeError):
    pass


@dataclass
class Communicator:
    group: Optional[dist.ProcessGroup]   # None = the default (world) group
    rank: int
    world_size: int
    device: torch.device

    @property
    def backend(self) -> str:
        return dist.get_backend(self.group)


def init_communicator(rank: int, world_size: int, init_method: str, device: torch.device,
                      timeout_s: float = 600.0) -> Communicator:
    """Creates the world communicator.  ``init_method`` is a ``tcp://ip:port`` rendezvous address."""
    backend = "nccl" if device.type == "cuda" else "gloo"
    kwargs = {}
    if device.type == "cuda":
        torch.cuda.set_device(device)
        kwargs["device_id"] = device
    try:
        dist.init_process_group(backend, init_method=init_method, rank=rank, world_size=world_size,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    except Exception as ex:  # noqa: BLE001
        raise CclError(f"communicator initialisation failed for rank {rank}/{world_size}: {ex}") from ex
    comm = Communicator(None, rank, world_size, device)
    barrier(comm)
    return comm


def world_communicator(device: torch.device) -> Communicator:
    """Wraps an already initialised default process group."""
    return Communicator(None, dist.get_rank(), dist.get_world_size(), device)


def create_subset_communicator(parent: Communicator, ranks: Sequence[int]) -> Optional[Communicator]:
    """Collective over the parent: every rank calls it; ranks outside ``ranks`` receive None
    (the reference's ``ncclCommSplit`` with ``NCCL_SPLIT_NOCOLOR``)."""
    group = dist.new_group(ranks=list(ranks))
    if parent.rank not in ranks:
        return None
    return Communicator(group, list(ranks).index(parent.rank), len(ranks), parent.device)


def destroy(comm: Communicator) -> None:
    """Destroys the communicator; falls back to abort when the orderly path fails."""
    try:
        if comm.group is None:
            dist.destroy_process_group()
        else:
            dist.destroy_process_group(comm.group)
    except Exception:  # noqa: BLE001
        abort(comm)


def abort(comm: Communicator) -> None:
    pg = comm.group if comm.group is not None else dist.group.WORLD
    try:
        backend = pg._get_backend(comm.device)  # type: ignore[attr-defined]
        if hasattr(backend, "abort"):
            backend.abort()
            return
    except Exception:  # noqa: BLE001
        pass
    try:
        dist.destroy_process_group(comm.group)
    except Exception:  # noqa: BLE001
        pass


def _global(comm: Communicator, rank_in_comm: int) -> int:
    return rank_in_comm if comm.group is None else dist.get_global_rank(comm.group, rank_in_comm)


def barrier(comm: Communicator) -> None:
    t = torch.ones(1, dtype=torch.int32, device=comm.device)
    try:
        dist.all_reduce(t, group=comm.group)
    except Exception as ex:  # noqa: BLE001
        raise CclError(f"barrier failed: {ex}") from ex
    if int(t.item()) != comm.world_size:
        raise CclError(f"barrier saw {int(t.item())} participants, expected {comm.world_size}")


def send_string(comm: Communicator, text: str, dst: int) -> None:
    raw = text.encode("utf-8")
    if len(raw) >= STRING_BYTES:
        raise CclError(f"string longer than {STRING_BYTES - 1} bytes")
    buf = torch.zeros(STRING_BYTES, dtype=torch.uint8)
    buf[:len(raw)] = torch.tensor(list(raw), dtype=torch.uint8)
    dist.send(buf.to(comm.device), _global(comm, dst), group=comm.group)


def recv_string(comm: Communicator, src: int) -> str:
    buf = torch.zeros(STRING_BYTES, dtype=torch.uint8, device=comm.device)
    dist.recv(buf, _global(comm, src), group=comm.group)
    raw = bytes(buf.cpu().tolist())
    return raw.split(b"\x00", 1)[0].decode("utf-8")


def send_buffer_async(comm: Communicator, tensor: torch.Tensor, dst: int):
    return dist.isend(tensor, _global(comm, dst), group=comm.group)


def recv_buffer_async(comm: Communicator, tensor: torch.Tensor, src: int):
    return dist.irecv(tensor, _global(comm, src), group=comm.group)


def broadcast_async(comm: Communicator, tensor: torch.Tensor, root: int):
    return dist.broadcast(tensor, _global(comm, root), group=comm.group, async_op=True)


_SUM_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.int32, torch.int64, torch.float64)


def all_reduce_async(comm: Communicator, tensor: torch.Tensor):
    if tensor.dtype not in _SUM_DTYPES:
        raise CclError(f"all-reduce does not support {tensor.dtype}")
    return dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=comm.group, async_op=True)


def all_gather_async(comm: Communicator, out: torch.Tensor, shard: torch.Tensor):
    return dist.all_gather_into_tensor(out, shard, group=comm.group, async_op=True)


def reduce_scatter_async(comm: Communicator, out_shard: torch.Tensor, full: torch.Tensor):
    return dist.reduce_scatter_tensor(out_shard, full, op=dist.ReduceOp.SUM, group=comm.group, async_op=True)
