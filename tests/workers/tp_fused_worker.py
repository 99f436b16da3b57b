"""Child process of the two-GPU tensor-parallel test: the block with fused all-gather→GEMM / GEMM→reduce-scatter
kernels must agree with the same block on NCCL collectives (output, input gradient, weight gradients)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main(out_path: str) -> None:
    from fbamtrain_b200.models.blocks import AttentionBlock
    from fbamtrain_b200.models.init_utils import SeedSequence
    from fbamtrain_b200.ops import native
    from fbamtrain_b200.parallel.tensor_parallel import TensorParallelBlock, TpContext, sync_replicated_grads
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    b, t, e, heads, mlp = 2, 384, 256, 4, 1024
    full = AttentionBlock(e, heads, mlp, True, True, 1e-5, torch.bfloat16, SeedSequence(3)).to(dev)
    x = torch.randn(b * t, e, device=dev).bfloat16()
    g = torch.randn(b * t, e, device=dev).bfloat16()
    rows = b * t // world
    results = {}
    for transport in ("nccl", "fused"):
        tp = TpContext(None, dev, transport)
        blk = TensorParallelBlock(full, tp, b, t).to(dev)
        xs = x[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
        for _ in range(2):                         # twice: the second pass reuses the staging windows
            for p in blk.parameters():
                p.grad = None
            xs.grad = None
            ys = blk(xs)
            ys.backward(g[rank * rows:(rank + 1) * rows])
        sync_replicated_grads([blk], tp)
        native.check_status(dev)
        torch.cuda.synchronize()
        results[transport] = [ys.detach().float(), xs.grad.float()] + [p.grad.float() for p in blk.parameters()]
    msg = "ok"
    for i, (a, c) in enumerate(zip(results["nccl"], results["fused"])):
        err = float((a - c).norm() / (a.norm() + 1e-6))
        if not err < 2e-2:
            msg = f"rank {rank}: tensor {i} differs (relative error {err})"
            break
    gathered = [None] * world
    dist.all_gather_object(gathered, msg)
    if rank == 0:
        bad = [m for m in gathered if m != "ok"]
        with open(out_path, "w") as f:
            f.write(bad[0] if bad else "ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
