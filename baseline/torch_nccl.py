#!/usr/bin/env python
"""Library baseline: the same model, optimizer and data as ``bench.py`` through plain PyTorch operators
(cuBLAS GEMMs, cuDNN convolutions and LSTM, library flash attention) with NCCL collectives for data parallelism
(all-reduce, or reduce-scatter + sharded AdamW + all-gather).  It stands in for the reference trainer's own
NCCL + cuBLAS build, which cannot be built offline, and is the number every fused path is compared against.

    python baseline/torch_nccl.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nproc-per-node 8 baseline/torch_nccl.py --gpus 8 --dp-mode zero1

Prints one JSON line in the format of ``bench.py`` with ``"impl": "torch_nccl_baseline"``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="fbam_small")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--frame-chunk", type=int, default=1024)
    ap.add_argument("--dp-mode", default="zero1", choices=["allreduce", "zero1"])
    a = ap.parse_args()
    import torch.distributed as dist
    from fbamtrain_b200 import RunConfiguration, Trainer, ops, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    import bench as B

    ops.set_backend("torch")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dp = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        from fbamtrain_b200.parallel.dp import DataParallel
        dp = DataParallel(mode=a.dp_mode)
    cfg = RunConfiguration.from_json(presets.PRESETS[a.model](a.micro_batch, world))
    if a.seq:
        cfg.train_sequence_length = a.seq
    seq = cfg.train_sequence_length
    trainer = Trainer(cfg, device=device, dp=dp, frame_chunk=a.frame_chunk)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, trainer.vocab,
                               seed=1000 + rank)
    batches = [tuple(t.to(device) for t in src.next_batch(a.micro_batch, seq)) for _ in range(2)]
    for i in range(max(3, a.warmup)):
        trainer.train_step(*batches[i % 2])
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = B.ClockSampler(local)
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(a.steps):
        loss = trainer.train_step(*batches[i % 2])
    end.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end)], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    trainer.logger.drain()
    if rank == 0:
        frames = a.micro_batch * seq * world
        flops = B.model_flops_per_step(cfg, a.micro_batch, seq)
        step_s = float(ms) / 1e3 / a.steps
        print(json.dumps({
            "metric": "train frames/sec", "value": frames / step_s, "unit": "frames/s", "n_gpus": world,
            "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "weak", "dtype": "bf16", "impl": "torch_nccl_baseline",
            "data": "synthetic seeded frames/actions, random-init weights", "mfu": flops / step_s / 2.25e15,
            "final_loss": float(loss),
            "config": {"model": a.model, "global_batch": a.micro_batch * world, "seq_len": seq,
                       "parallelism": f"dp{world}" + (f"-nccl-{a.dp_mode}" if world > 1 else ""),
                       "operators": "cuBLAS / cuDNN conv + LSTM / SDPA flash"},
            "clocks": clocks}))
    trainer.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
