"""Two ranks under torchrun, each with the default NCCL group AND a stand-alone ScopedGroup next to it (the
communicator that same-position ranks of different pipelines use): sum, broadcast and object exchange on it, then a
collective on the default group to show that it was left alone.  NVLink multicast stays out (a member of such a group
may vanish)."""
import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from fbamtrain_b200.parallel.ftccl import (ScopedGroup, SharedStateSyncStrategy, TensorInfo, Result,
                                           synchronize_shared_state)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    device = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    port = int(sys.argv[2])
    group = ScopedGroup("127.0.0.1", port, host_store=rank == 0, prefix="test/1/0", rank=rank, world_size=world,
                        device=device, timeout_s=60.0)
    x = torch.full((1 << 20,), float(rank + 1), device=device)
    group.all_reduce(x)
    assert float(x[0]) == sum(range(1, world + 1)) and float(x[-1]) == float(x[0])
    y = torch.full((1000,), float(rank), device=device)
    group.broadcast(y, src=world - 1)
    assert float(y.sum()) == 1000.0 * (world - 1)
    got = group.all_gather_object({"rank": rank, "name": "x" * (rank * 7)})
    assert [g["rank"] for g in got] == list(range(world)) and len(got[1]["name"]) == 7
    # shared state: rank 1 is a revision ahead, so its content wins
    t = torch.full((4096,), float(rank), device=device, dtype=torch.bfloat16)
    res, info = synchronize_shared_state(group, 5 + rank, [TensorInfo("t", t)], SharedStateSyncStrategy.ENFORCE_POPULAR)
    assert res == Result.SUCCESS and info.revision == 6 and float(t.float().mean()) == 1.0
    z = torch.ones(8, device=device)
    dist.all_reduce(z)                                   # the default group still works
    assert float(z[0]) == world
    torch.cuda.synchronize()
    group.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        open(sys.argv[1], "w").write("ok")


if __name__ == "__main__":
    main()
