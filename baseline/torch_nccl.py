#!/usr/bin/env python
"""Library baseline — NOT the reference trainer: the FBAM benchmark model written directly against PyTorch's own
operators, the way one would write it without this package.

    python baseline/torch_nccl.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 baseline/torch_nccl.py --gpus 8

Everything on the hot path is a vendor-library kernel in its favourable configuration: bf16 autocast over fp32
parameters, channels-last cuDNN convolutions, ``F.gelu`` / ``F.rms_norm`` on bf16 tensors, ``nn.LSTM`` with
flattened cuDNN weights, ``F.scaled_dot_product_attention`` (flash), ``F.cross_entropy``, ``torch.optim.AdamW(fused=True)``
and, for more than one GPU, ``DistributedDataParallel`` over NCCL.  Same architecture, shapes, data and loss
normalisation as ``bench.py`` (FBAM-small / FBAM-1B presets); the optimizer is AdamW for both (PyTorch has no Muon).
It answers "what does the same model cost on library kernels on this GPU"; the reference itself (a C++ binary with
ahead-of-time compiled kernels) cannot be built offline.

Prints one JSON line in the format of ``bench.py`` with ``"impl": "torch_library_baseline"``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class Block(nn.Module):
    def __init__(self, dim, heads, mlp):
        super().__init__()
        self.heads = heads
        self.g1 = nn.Parameter(torch.ones(dim))
        self.g2 = nn.Parameter(torch.ones(dim))
        self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.fc1, self.fc2 = nn.Linear(dim, mlp), nn.Linear(mlp, dim)

    def forward(self, x):
        b, t, e = x.shape
        q, k, v = self.qkv(F.rms_norm(x, (e,), self.g1.to(x.dtype), 1e-5)).view(b, t, 3, self.heads, e // self.heads).unbind(2)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.proj(o.transpose(1, 2).reshape(b, t, e))
        return x + self.fc2(F.gelu(self.fc1(F.rms_norm(x, (e,), self.g2.to(x.dtype), 1e-5))))


class LibraryFbam(nn.Module):
    def __init__(self, m, vocab):
        super().__init__()
        self.rows, self.cols = m.frame_rows, m.frame_cols
        e = m.embed_dim
        self.cp = nn.Embedding(m.max_code_point, e)
        self.pos = nn.Parameter(torch.randn(self.rows * self.cols, e))
        self.colour = nn.Parameter(torch.randn(6, e))
        chans = list(m.block_channels())
        self.convs = nn.ModuleList([nn.Conv2d(ci, co, 3, stride=2, padding=1, bias=False) for ci, co in chans])
        self.proj = nn.Linear(chans[-1][1], m.n_embed)
        self.lstm = nn.LSTM(m.n_embed, m.hidden, num_layers=m.lstm_layers, batch_first=True)
        self.blocks = nn.ModuleList([Block(m.hidden, m.action_heads, m.action_mlp_dim or 4 * m.hidden)
                                     for _ in range(m.action_blocks)])
        self.gf = nn.Parameter(torch.ones(m.hidden))
        self.head = nn.Linear(m.hidden, vocab, bias=False)
        self.vocab = vocab

    def frame_head(self, cells):                              # (N, P, 3) int32 -> (N, n_embed)
        n = cells.shape[0]
        cp = cells[..., 0].long().clamp(0, self.cp.num_embeddings - 1)
        fg, bg = cells[..., 1], cells[..., 2]
        ch = torch.stack([(fg >> 16) & 255, (fg >> 8) & 255, fg & 255, (bg >> 16) & 255, (bg >> 8) & 255, bg & 255],
                         -1).to(torch.bfloat16) / 255.0
        x = self.cp(cp) + self.pos + ch @ self.colour.to(torch.bfloat16)
        x = x.to(torch.bfloat16).view(n, self.rows, self.cols, -1).permute(0, 3, 1, 2)   # NCHW view, channels-last memory
        for conv in self.convs:
            x = F.gelu(conv(x))
        return self.proj(x.mean(dim=(2, 3)))

    def forward(self, cells, targets, scale, chunk):
        b, t, p, _ = cells.shape
        flat = cells.view(b * t, p, 3)
        emb = torch.cat([self.frame_head(flat[i:i + chunk]) for i in range(0, b * t, chunk)], 0).view(b, t, -1)
        h, _ = self.lstm(emb)
        for blk in self.blocks:
            h = blk(h)
        logits = self.head(F.rms_norm(h, (h.shape[-1],), self.gf.to(h.dtype), 1e-5))
        return F.cross_entropy(logits.float().view(b * t, -1), targets.view(-1), reduction="sum") * scale


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="fbam_small")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--frame-chunk", type=int, default=1024)
    a = ap.parse_args()
    import torch.distributed as dist
    from fbamtrain_b200 import RunConfiguration, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    import bench as B

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    cfg = RunConfiguration.from_json(presets.PRESETS[a.model](a.micro_batch, world))
    if a.seq:
        cfg.train_sequence_length = a.seq
    seq = cfg.train_sequence_length
    m = cfg.model_config
    vocab = m.action_vocab
    torch.manual_seed(0)
    model = LibraryFbam(m, vocab).to(device).to(memory_format=torch.channels_last)
    model.lstm.flatten_parameters()
    net = nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=cfg.optimizer_config.learning_rate,
                            weight_decay=cfg.optimizer_config.weight_decay, fused=True)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, m.max_code_point, vocab, seed=1000 + rank)
    batches = [tuple(t.to(device) for t in src.next_batch(a.micro_batch, seq)) for _ in range(2)]
    scale = 1.0 / (seq * a.micro_batch * world)

    def step(i):
        cells, targets = batches[i % 2]
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(cells, targets, scale, a.frame_chunk)
        loss.backward()
        opt.step()
        return loss

    for i in range(max(3, a.warmup)):
        step(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = B.ClockSampler(local)
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(a.steps):
        loss = step(i)
    end.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end)], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        frames = a.micro_batch * seq * world
        flops = B.model_flops_per_step(cfg, a.micro_batch, seq)
        step_s = float(ms) / 1e3 / a.steps
        print(json.dumps({
            "metric": "train frames/sec", "value": frames / step_s, "unit": "frames/s", "n_gpus": world,
            "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "weak", "dtype": "bf16 autocast, fp32 parameters", "impl": "torch_library_baseline",
            "note": "library baseline written against PyTorch operators; not the reference trainer",
            "data": "synthetic seeded frames/actions, random-init weights", "mfu": flops / step_s / 2.25e15,
            "final_loss": float(loss), "peak_memory_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
            "config": {"model": a.model, "global_batch": a.micro_batch * world, "seq_len": seq,
                       "parallelism": f"dp{world}" + ("-ddp-nccl" if world > 1 else ""), "optimizer": "adamw (fused)",
                       "operators": "cuDNN channels-last conv / cuDNN LSTM / SDPA flash / cuBLAS / fused AdamW"},
            "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
