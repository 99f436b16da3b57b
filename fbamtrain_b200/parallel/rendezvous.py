"""TCP rendezvous that hands every rank the communicator bootstrap blob.

Protocol of the reference (reference: ``src/rdvz.cpp:48-116, 118-206``): rank 0 listens on the
``ip:port`` of the parallel configuration; every other rank connects (up to 50 attempts, 100 ms
apart), sends its rank as a little-endian u32 and receives a fixed 128-byte blob; ranks that are out
of range or appear twice are rejected and the rendezvous fails.  In the reference the blob is the
NCCL unique id; here it is the address of the store that ``torch.distributed`` bootstraps from
(``tcp://ip:port`` plus a random token), zero-padded to 128 bytes — NCCL's own id exchange then runs
through that store.  ``perform_ccl_rendezvous`` does the exchange and creates the communicator.
"""
from __future__ import annotations

import os
import socket
import struct
import time
from typing import Optional

import torch

from . import ccl

BLOB_BYTES = 128
CONNECT_RETRIES = 50
RETRY_DELAY_S = 0.1


class RendezvousError(RuntimeError):
    pass


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    data = b""
    while len(data) < n:
        chunk = sock.recv(n - len(data))
        if not chunk:
            raise RendezvousError("peer closed the connection during rendezvous")
        data += chunk
    return data


def serve_blob(ip: str, port: int, world_size: int, blob: bytes, timeout_s: float = 60.0) -> None:
    """Rank 0: accept ``world_size - 1`` peers and send each the blob."""
    if len(blob) != BLOB_BYTES:
        raise ValueError(f"blob must be {BLOB_BYTES} bytes")
    srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    try:
        srv.bind((ip, port))
        srv.listen(max(1, world_size))
        srv.settimeout(timeout_s)
        seen = {0}
        conns = []
        try:
            while len(seen) < world_size:
                try:
                    conn, _ = srv.accept()
                except socket.timeout as ex:
                    raise RendezvousError(f"rendezvous timed out with ranks {sorted(seen)} present") from ex
                conn.settimeout(timeout_s)
                (rank,) = struct.unpack("<I", _recv_exact(conn, 4))
                if rank == 0 or rank >= world_size:
                    conn.close()
                    raise RendezvousError(f"rank {rank} is out of range for world size {world_size}")
                if rank in seen:
                    conn.close()
                    raise RendezvousError(f"rank {rank} connected twice")
                seen.add(rank)
                conns.append(conn)
            for conn in conns:
                conn.sendall(blob)
        finally:
            for conn in conns:
                conn.close()
    finally:
        srv.close()


def fetch_blob(ip: str, port: int, rank: int, timeout_s: float = 60.0) -> bytes:
    last: Optional[Exception] = None
    for _ in range(CONNECT_RETRIES):
        try:
            with socket.create_connection((ip, port), timeout=timeout_s) as sock:
                sock.sendall(struct.pack("<I", rank))
                return _recv_exact(sock, BLOB_BYTES)
        except (ConnectionRefusedError, ConnectionResetError, socket.timeout, OSError) as ex:
            last = ex
            time.sleep(RETRY_DELAY_S)
    raise RendezvousError(f"could not reach the rendezvous at {ip}:{port}: {last}")


def _free_port(ip: str) -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((ip, 0))
        return s.getsockname()[1]


def perform_ccl_rendezvous(ip: str, port: int, rank: int, world_size: int, device: torch.device,
                           timeout_s: float = 60.0) -> ccl.Communicator:
    """Exchanges the bootstrap blob and returns the world communicator (reference:
    ``include/rdvz.h:19-26``, ``src/rdvz.cpp:241-298``)."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise RendezvousError(f"rank {rank} is out of range for world size {world_size}")
    if rank == 0:
        store_port = _free_port(ip)
        text = f"tcp://{ip}:{store_port}#{os.urandom(4).hex()}".encode("ascii")
        blob = text + b"\x00" * (BLOB_BYTES - len(text))
        if world_size > 1:
            serve_blob(ip, port, world_size, blob, timeout_s)
    else:
        blob = fetch_blob(ip, port, rank, timeout_s)
    address = blob.split(b"\x00", 1)[0].decode("ascii").split("#", 1)[0]
    return ccl.init_communicator(rank, world_size, address, device, timeout_s=max(timeout_s, 60.0))


def teardown(comm: ccl.Communicator) -> None:
    """Destroy, falling back to abort (reference: ``src/rdvz.cpp:267-285``)."""
    ccl.destroy(comm)
