"""Child process of the multi-GPU data-parallel test (launched with torch.distributed.run).

Trains the tiny bf16 model for a few steps with the fused peer-memory path and with the NCCL
reduce-scatter / all-gather path from identical initial weights and data, and checks that both give
the same parameters on every rank.  Writes ``ok`` or the mismatch to the file named on the command line.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main(out_path: str, multicast: bool, optimizer: str = "adamw", transport: str = "symm") -> None:
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.ops import native
    from fbamtrain_b200.parallel.dp import DataParallel
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    d = presets.tiny("bf16")
    d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64], "n_embed": 64})
    d["micro_batch_size"], d["total_batch_size"] = 2, 2 * world
    d["optimizer"]["type"] = optimizer
    cfg = RunConfiguration.from_json(d)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=100 + rank, pin=False)
    batches = [src.next_batch(2, cfg.train_sequence_length) for _ in range(3)]
    results = {}
    for mode in ("zero1", "fused"):
        tr = Trainer(cfg, device=dev, dp=DataParallel(mode=mode, use_multicast=multicast and mode == "fused",
                                                      window_transport=transport))
        losses = [float(tr.train_step(c, t)) for c, t in batches]
        native.check_status(dev)
        torch.cuda.synchronize()
        results[mode] = ({n: p.detach().float().clone() for n, p in tr.model.named_parameters()}, losses)
        tr.close()
    msg = "ok"
    for n, p in results["zero1"][0].items():
        q = results["fused"][0][n]
        if "qkv.bias" in n:
            continue
        if not torch.allclose(p, q, atol=2e-2, rtol=2e-2):
            msg = f"rank {rank}: parameter {n} differs by {float((p - q).abs().max())}"
            break
    if abs(results["zero1"][1][-1] - results["fused"][1][-1]) > 5e-2:
        msg = f"rank {rank}: losses differ {results['zero1'][1]} vs {results['fused'][1]}"
    # every rank must hold identical parameters after the fused all-gather
    for n, q in results["fused"][0].items():
        ref = q.clone()
        dist.broadcast(ref, src=0)
        if not torch.equal(ref, q):
            msg = f"rank {rank}: parameter {n} is not identical to rank 0's"
            break
    gathered = [None] * world
    dist.all_gather_object(gathered, msg)
    if rank == 0:
        bad = [m for m in gathered if m != "ok"]
        with open(out_path, "w") as f:
            f.write(bad[0] if bad else "ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], "multicast" in sys.argv[2:], "muon" if "muon" in sys.argv[2:] else "adamw",
         "ipc" if "ipc" in sys.argv[2:] else "symm")
