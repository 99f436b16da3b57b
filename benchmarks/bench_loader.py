#!/usr/bin/env python
"""Host-side batch assembly throughput: the native loader (memory-mapped ``.fbrec`` recordings, worker threads)
against the per-frame Python path, at the frame geometry of the benchmark model.  No GPU involved.

    python benchmarks/bench_loader.py [--rows 48 --cols 160 --frames 2048 --batch 8 --seq 1024 --threads 8]

Prints one JSON line: frames/s and GB/s of both paths.  A training step of the small benchmark model consumes
8 x 1024 frames (755 MB of cell states) per GPU every ≈ 0.12 s, i.e. ≈ 70 k frames/s or 6.4 GB/s per GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=48)
    ap.add_argument("--cols", type=int, default=160)
    ap.add_argument("--frames", type=int, default=2048)
    ap.add_argument("--recordings", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--threads", type=int, default=8)
    ap.add_argument("--python-positions", type=int, default=512, help="positions to time on the Python path")
    a = ap.parse_args()
    from fbamtrain_b200 import runtime as rt
    from fbamtrain_b200.data.iterator import Batch
    from fbamtrain_b200.data.recording import RawRecording, write_raw_recording
    from fbamtrain_b200.tokenizer import Tokenizer
    from fbamtrain_b200.train import build_batch_from_recordings
    rng = np.random.default_rng(0)
    tok = Tokenizer(list("abcdefghijklmnopqrstuvwxyz") + ["th", "he", "in", "er"])
    with tempfile.TemporaryDirectory() as d:
        paths = []
        for r in range(a.recordings):
            cells = rng.integers(0, 512, size=(a.frames, a.rows, a.cols, 3), dtype=np.uint32)
            keys = ["abcdefghijklmnopqrstuvwxyz"[int(i)] for i in rng.integers(0, 26, size=a.frames)]
            path = os.path.join(d, f"r{r}.fbrec")
            write_raw_recording(path, cells, keys)
            paths.append(path)
        loader = rt.NativeBatchLoader(paths, tok.tokens, 512, 4096, threads=a.threads)
        cells_out = torch.empty((a.batch, a.seq, a.rows * a.cols, 3), dtype=torch.int32)
        targets_out = torch.empty((a.batch, a.seq), dtype=torch.int64)
        indices = [int(i) for i in rng.integers(0, a.recordings, size=a.batch)]
        starts = [int(s) for s in rng.integers(0, max(1, a.frames - a.seq), size=a.batch)]
        loader.fill(indices, starts, a.seq, cells_out, targets_out)       # warm the page cache and the buffers
        times = []
        for _ in range(5):
            t0 = time.perf_counter()
            loader.fill(indices, starts, a.seq, cells_out, targets_out)
            times.append(time.perf_counter() - t0)
        native_s = sorted(times)[len(times) // 2]
        recs = [RawRecording(p) for p in paths]
        py_seq = max(1, a.python_positions // a.batch)
        t0 = time.perf_counter()
        build_batch_from_recordings(Batch([recs[i] for i in indices], indices, starts), tok, py_seq, a.rows, a.cols,
                                    4096, 512)
        python_s = time.perf_counter() - t0
    frame_bytes = a.rows * a.cols * 12
    out = {"bench": "batch_loader", "rows": a.rows, "cols": a.cols, "batch": a.batch, "seq": a.seq,
           "threads": a.threads,
           "native_frames_per_s": a.batch * a.seq / native_s, "native_gb_per_s": a.batch * a.seq * frame_bytes / native_s / 1e9,
           "python_frames_per_s": a.batch * py_seq / python_s,
           "python_gb_per_s": a.batch * py_seq * frame_bytes / python_s / 1e9,
           "speedup": (a.batch * a.seq / native_s) / (a.batch * py_seq / python_s)}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
