#!/usr/bin/env python
"""Where one training step spends its GPU time: kernel totals, the collective kernels on the timeline, idle gaps.

    python benchmarks/step_timeline.py                                   # one GPU
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/step_timeline.py   # fused DP

Runs the ``bench.py`` configuration (FBAM-small, micro-batch 8 x 1024 frames per GPU, fused data parallelism for more
than one rank), warms up, records ONE step with the PyTorch profiler (CUPTI kernel records: the numbers are kernel
durations, not wall-clock shares) and prints, for rank 0: the span of the step, the union of all kernel intervals
("GPU busy"), the kernels of the fused reduce-scatter + AdamW + all-gather path with their start times, idle gaps
longer than 0.1 ms, and the kernel totals (``FBAMTRAIN_PROFILE_LABELS=1`` adds the op labels of the launchers).
A profiled step is a few per cent slower than an unprofiled one; use ``bench.py`` for the step time itself.
"""
from __future__ import annotations

import os
import sys

os.environ.setdefault("FBAMTRAIN_PROFILE_LABELS", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main() -> None:
    from torch.profiler import ProfilerActivity, profile
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dp = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        from fbamtrain_b200.parallel.dp import DataParallel
        dp = DataParallel(mode="fused")
    micro = 8
    cfg = RunConfiguration.from_json(presets.fbam_small(micro, world))
    trainer = Trainer(cfg, device=device, dp=dp, frame_chunk=1024)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, trainer.vocab,
                               seed=1000 + rank)
    cells, targets = src.next_batch(micro, cfg.train_sequence_length)
    cells, targets = cells.to(device), targets.to(device)
    for _ in range(3):
        trainer.train_step(cells, targets)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        trainer.train_step(cells, targets)
        torch.cuda.synchronize()
    if rank == 0:
        kernels = sorted((e for e in prof.events() if e.device_type.name == "CUDA"), key=lambda e: e.time_range.start)
        t0 = kernels[0].time_range.start
        t1 = max(e.time_range.end for e in kernels)
        busy, cur_s, cur_e, gaps = 0, None, None, []
        for e in kernels:
            s, en = e.time_range.start, e.time_range.end
            if cur_e is None or s > cur_e:
                if cur_e is not None:
                    busy += cur_e - cur_s
                    if s - cur_e > 100:
                        gaps.append((cur_e - t0, s - cur_e, e.name))
                cur_s, cur_e = s, en
            else:
                cur_e = max(cur_e, en)
        busy += cur_e - cur_s
        print(f"ranks {world}; step span {(t1 - t0) / 1e3:.2f} ms; GPU busy (union of kernel intervals) {busy / 1e3:.2f} ms")
        print("collective kernels (start, duration):")
        for e in kernels:
            if any(k in e.name for k in ("rs_adamw", "peer_barrier", "reduce_pull", "push_shard", "nccl")):
                print(f"  {(e.time_range.start - t0) / 1e3:8.3f} ms  +{(e.time_range.end - e.time_range.start) / 1e3:6.3f} ms  {e.name[:70]}")
        print("idle gaps > 0.1 ms (start, length, next kernel):")
        for start, length, name in gaps:
            print(f"  {start / 1e3:8.3f} ms  {length / 1e3:6.3f} ms  {name[:60]}")
        rows = sorted(((e.key, e.device_time_total / 1e3, e.count) for e in prof.key_averages() if e.device_time_total > 0),
                      key=lambda r: -r[1])
        print("totals (kernels, and the launchers' labels which contain them):")
        for key, ms, count in rows[:45]:
            print(f"  {ms:8.3f} ms  x{count:<4d} {key[:100]}")
    trainer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
