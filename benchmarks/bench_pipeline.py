"""Two-stage pipeline benchmark: frame head on the first half of the ranks, action model (tensor-parallel
attention / MLP blocks, replicated LSTM) on the second half, NCCL point-to-point between partner ranks.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_pipeline.py \
        [--model fbam_1b] [--micro-batches 8] [--mb-size 2] [--seq 2048] [--tp fused|nccl] [--steps 3]

One step = all micro-batches forward and backward through both stages, the gradient all-reduces inside each stage
and the optimizer step of every rank's parameters.  Rank 0 prints one JSON line; the time is the CUDA-event time
of the timed steps, maximum over ranks.  The closest mode of the reference is its frame-head parallelism
(``src/main.cpp:3119-3123, 3204-3273``), which has no published throughput.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
# few CTAs per send/receive kernel: they share the GPU with persistent compute kernels (see parallel/pipeline.py)
os.environ.setdefault("NCCL_MAX_P2P_NCHANNELS", "4")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="fbam_1b", choices=["fbam_small", "fbam_1b"])
    ap.add_argument("--micro-batches", type=int, default=8)
    ap.add_argument("--mb-size", type=int, default=2)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--tp", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2 or world % 2:
        raise SystemExit("launch with torch.distributed.run on an even number of GPUs")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)

    from fbamtrain_b200 import RunConfiguration, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.models import FbamModel
    from fbamtrain_b200.ops import native
    from fbamtrain_b200.optim import create_optimizer
    from fbamtrain_b200.parallel.pipeline import PipelineLayout, TwoStagePipeline

    cfg = RunConfiguration.from_json(presets.PRESETS[a.model](a.mb_size, 1))
    seq = a.seq or cfg.train_sequence_length
    vocab = cfg.model_config.action_vocab
    torch.manual_seed(0)
    model = FbamModel(cfg.model_config, vocab).to(dev)
    pipe = TwoStagePipeline(model, PipelineLayout.even_split(world), dev, a.micro_batches, a.mb_size, seq, a.tp)
    named = [(f"p{i}", p) for i, p in enumerate(pipe.parameters_of_stage())]
    opt = create_optimizer(cfg.optimizer_config, named, "frame_head" if pipe.is_frame else "action_model")

    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, vocab, seed=7, pin=False)
    one_cells, one_targets = src.next_batch(a.mb_size, seq)            # the same micro-batch is replayed
    cells = one_cells.to(dev).unsqueeze(0).expand(a.micro_batches, *one_cells.shape)
    cells = cells.reshape(a.micro_batches, a.mb_size, seq, -1, 3) if cells.dim() != 5 else cells
    targets = one_targets.to(dev).unsqueeze(0).expand(a.micro_batches, *one_targets.shape)
    scale = 1.0 / (seq * a.micro_batches * a.mb_size)

    def step():
        for _, p in named:
            p.grad = None
        loss = pipe.run_step(cells if pipe.is_frame else None, None if pipe.is_frame else targets, scale)
        opt.step()
        return loss

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    launches0 = native.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss = 0.0
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    lt = torch.tensor([loss], device=dev)
    dist.all_reduce(lt)
    frames = a.micro_batches * a.mb_size * seq
    if rank == 0:
        print(json.dumps({
            "bench": "two_stage_pipeline", "model": a.model, "n_gpus": world, "tp_transport": a.tp,
            "micro_batches": a.micro_batches, "micro_batch_size": a.mb_size, "seq_len": seq,
            "ms_per_step": float(t.item()), "frames_per_s": frames / (float(t.item()) / 1e3),
            "loss": float(lt.item()), "optimizer": cfg.optimizer_config.type, "dtype": "bf16",
            "gpu_launches_rank0": native.launches() - launches0,
            "p2p_bytes_rank0_per_step": pipe.stats["p2p_bytes"] // (a.warmup + a.steps),
            "data": "synthetic seeded frames/actions (one micro-batch replayed), random-init weights"}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
