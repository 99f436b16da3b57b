#!/usr/bin/env python
"""Headline benchmark: training throughput (frames/s) and MFU of FBAM-small, bf16, AdamW, pure data
parallel, sequence 1024 frames, micro-batch 8 per GPU, synthetic seeded frames and random-init weights.

    python bench.py --gpus N --steps K --warmup W          # N > 1: launched under torch.distributed.run

Two numbers are measured with CUDA events (max over ranks):

* ``value`` — K optimizer steps with the batch already resident on the device;
* ``e2e.value`` — K calls of the public ``Trainer.train_step`` with host inputs: every step uploads its
  frames and targets from pinned host memory and reads the step loss back to the host.

``--impl reference`` would run the unmodified reference trainer; it cannot be built offline (see
``reference_unavailable_reason``), so that arm prints an ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_FRAMES_PER_SEC = None  # the reference publishes no end-to-end throughput


def reference_unavailable_reason() -> str:
    return ("reference is a CMake/C++ binary, not a Python package: `pip install --no-index ... <reference checkout>` fails "
            "with \"Neither 'setup.py' nor 'pyproject.toml' found\"; its six git submodules (json, argparse, "
            "termstreamxz, threadpark, nccl, pccl) are empty and its kernels are fetched/AOT-built from the network")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def model_flops_per_step(cfg, batch: int, seq: int) -> float:
    """Useful FLOPs of one training step (forward + backward = 3 x forward matmul FLOPs)."""
    m = cfg.model_config
    frames = batch * seq
    h, w = m.frame_rows, m.frame_cols
    fwd = 0.0
    for cin, cout in m.block_channels():
        if m.downsample_conv_stride == 2:
            h, w = (h + 1) // 2, (w + 1) // 2
        mult = 2 if m.downsample_conv_mode == "geglu" else 1
        fwd += 2.0 * frames * h * w * cout * mult * cin * 9
        if m.downsample_conv_stride == 1:
            h, w = h // 2, w // 2
    feat = m.frame_feature_dim
    tokens_fh = h * w
    fwd += m.n_layer * frames * (2.0 * tokens_fh * 12 * feat * feat + 4.0 * tokens_fh * tokens_fh * feat)
    if m.frame_proj:
        fwd += 2.0 * frames * feat * m.n_embed
    hid = m.hidden
    for layer in range(m.lstm_layers):
        fwd += 2.0 * frames * ((m.n_embed if layer == 0 else hid) + hid) * 4 * hid
    mlp = m.action_mlp_dim or 4 * hid
    fwd += m.action_blocks * frames * (2.0 * (4 * hid * hid + 2 * hid * mlp) + 4.0 * seq * hid / 2)  # causal: half
    vocab = m.action_vocab
    fwd += 2.0 * frames * hid * vocab
    return 3.0 * fwd


def run_ours(args) -> dict:
    import torch.distributed as dist
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.ops import native
    from fbamtrain_b200.utils import flops as flops_counter
    from fbamtrain_b200.utils.mfu import measured_peaks, peak_tflops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dp = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        from fbamtrain_b200.parallel.dp import DataParallel
        dp = DataParallel(mode=args.dp_mode)

    micro = args.micro_batch
    cfg = RunConfiguration.from_json(presets.PRESETS[args.model](micro, world))
    cfg.model_config.dtype = args.dtype
    if args.seq:
        cfg.train_sequence_length = args.seq
    seq = cfg.train_sequence_length
    trainer = Trainer(cfg, device=device, dp=dp, frame_chunk=args.frame_chunk)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, trainer.vocab,
                               seed=1000 + rank)
    n_host = 2
    host_batches = [src.next_batch(micro, seq) for _ in range(n_host)]
    dev_batches = [(c.to(device), t.to(device)) for c, t in host_batches]
    h2d_bytes = host_batches[0][0].numel() * 4 + host_batches[0][1].numel() * 8

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(batches, read_loss: bool):
        for i in range(args.warmup):
            step_no = trainer.step_count
            trainer.train_step(*batches[i % len(batches)])
            if read_loss:
                trainer.host_loss(step_no)
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = native.launches()
        flops0 = flops_counter.snapshot()[0]
        clocks = None
        try:
            start.record()
            last = None
            previous = None
            for i in range(args.steps):
                step_no = trainer.step_count
                loss = trainer.train_step(*batches[i % len(batches)])
                if not read_loss:
                    last = loss
                    continue
                # end to end: every step's loss reaches the host inside the timed region, read one step late (after
                # the next step has been queued) the way a training loop logs it, so the host never drains the device
                if previous is not None:
                    last = trainer.host_loss(previous)
                previous = step_no
            if previous is not None:
                last = trainer.host_loss(previous)
            end.record()
            barrier()
            ms = start.elapsed_time(end)
        finally:
            if rank == 0:                       # the sampler is a child process: never leave it running
                clocks = sampler.stop()
        t = torch.tensor([ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        executed = flops_counter.snapshot()[0] - flops0
        return float(t.item()), clocks, float(last), native.launches() - launches0, executed

    def status_code() -> int:
        """0 unless a bounded device-side wait ran out on some rank (which would invalidate the measurement)."""
        word = native.status_word(device)
        code = torch.tensor([int(word.item())], device=device)
        word.zero_()
        if world > 1:
            dist.all_reduce(code, op=dist.ReduceOp.MAX)
        return int(code.item())

    ms_dev, clocks, last_loss, launches, executed_flops = timed(dev_batches, read_loss=False)
    status_dev = status_code()
    e2e_error = None
    try:
        ms_e2e, clocks_e2e, _, _, _ = timed(host_batches, read_loss=True)
    except Exception as ex:  # noqa: BLE001 - the device-timed result above is still reported
        e2e_error, ms_e2e, clocks_e2e = f"{type(ex).__name__}: {ex}", None, None
    status_e2e = status_code()
    trainer.logger.drain()

    frames_per_step = micro * seq * world
    value = frames_per_step * args.steps / (ms_dev / 1e3)
    e2e_value = frames_per_step * args.steps / (ms_e2e / 1e3) if ms_e2e else None
    flops = model_flops_per_step(cfg, micro, seq)
    peak = peak_tflops("B200", "bf16") * 1e12
    meas = measured_peaks()
    step_s = ms_dev / 1e3 / args.steps
    out = {
        "metric": "train frames/sec", "value": value, "unit": "frames/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / BASELINE_FRAMES_PER_SEC) if BASELINE_FRAMES_PER_SEC else None,
        "dtype": args.dtype, "data": "synthetic seeded frames/actions, random-init weights",
        "impl": "ours",
        "mfu": flops / step_s / peak,
        "mfu_of_measured_sustained_cublas": flops / step_s / (meas["bf16_tflops_sustained"] * 1e12),
        "peaks_source": meas["source"],
        "model_tflop_per_step_per_gpu": flops / 1e12,
        # "mfu" counts the arithmetic of the model as specified (dense 3x3 convolutions over the embedded cells).  The
        # fused first frame-head layer replaces that layer's three convolutions by table look-ups, so the tensor cores
        # execute fewer FLOPs than the model has: the executed count and its utilisation are given beside it.
        "executed_tflop_per_step_per_gpu": executed_flops / args.steps / 1e12,
        "hfu_executed_flops": executed_flops / args.steps / step_s / peak,
        "final_loss": last_loss,
        "config": {"model": args.model, "global_batch": micro * world, "micro_batch_per_gpu": micro, "seq_len": seq,
                   "parallelism": f"dp{world}" + (f"-{args.dp_mode}" if world > 1 else ""), "optimizer": cfg.optimizer_config.type,
                   "l2_policy": "inputs larger than L2 (≈0.75 GB of frames and >10 GB of activations per step)",
                   "frame_chunk": args.frame_chunk},
        "clocks": clocks,
        "e2e": {"error": e2e_error} if e2e_error else {
                "value": e2e_value, "unit": "frames/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "clocks": clocks_e2e,
                "api": "Trainer.train_step(pinned host cells, targets) + Trainer.host_loss(step); each step's loss is "
                       "read on the host after the next step has been queued, the last one before the timed region ends"},
        "gpu_launches": launches,
        "device_status": {"timed": status_dev, "e2e": status_e2e,
                          "meaning": "0 = no bounded device-side wait expired on any rank"},
    }
    trainer.close()
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="fbam_small", choices=["fbam_small", "fbam_1b"])
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--frame-chunk", type=int, default=1024)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"],
                    help="model / compute dtype (fp32 accumulation in both; the headline number is bf16)")
    ap.add_argument("--dp-mode", default="fused", choices=["allreduce", "zero1", "fused"])
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": reference_unavailable_reason()}))
        return
    out = run_ours(args)
    if out:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
