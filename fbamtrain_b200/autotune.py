"""Measures tile configurations for the GEMM / convolution shapes a model launches and writes a tuning table.

    python -m fbamtrain_b200.autotune --model fbam_small --micro-batch 8 --seq 1024 --out tuning.json
    FBAMTRAIN_TUNING_FILE=tuning.json python -m fbamtrain_b200.cli -c run.json ...

Step 1 runs one training step of the model with shape recording on (``ops.tuning.recording``): every tunable launch
reports its key and geometry.  Step 2 rebuilds each distinct launch on random operands and times every candidate
configuration with CUDA events (L2 flushed between iterations); a candidate the launcher rejects is skipped.  The
table format and the launcher side are described in ``ops/tuning.py``.  What the reference does with its autotune
drivers per architecture (reference: ``kernel_gen/kernel_gen/pysrc/autotune_matmul.py``,
``kernel_gen/kernel_gen/pysrc/autotune_conv2d.py``), for this package's kernels on the GPU at hand.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from typing import Callable, Dict, List, Optional

import torch

from .ops import tuning


def collect_shapes(model: str, micro_batch: int, seq: int, device: torch.device) -> Dict[str, dict]:
    """``{key: geometry}`` of the tunable launches of one training step."""
    from . import presets
    from .config import RunConfiguration
    from .data import SyntheticBatchSource
    from .train import Trainer
    cfg = RunConfiguration.from_json(getattr(presets, model)(micro_batch, 1))
    cfg.train_sequence_length = seq
    trainer = Trainer(cfg, device=device)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, trainer.vocab,
                               seed=0, pin=device.type == "cuda")
    cells, targets = src.next_batch(micro_batch, seq)
    with tuning.recording() as seen:
        trainer.train_step(cells, targets)
    trainer.close()
    return dict(seen)


def _time_ms(run: Callable[[], None], flush: torch.Tensor, warmup: int, iters: int) -> float:
    for _ in range(warmup):
        run()
    samples = []
    for _ in range(iters):
        flush.zero_()                                   # larger than L2: the operands come from HBM every time
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run()
        stop.record()
        stop.synchronize()
        samples.append(start.elapsed_time(stop))
    return statistics.median(samples)


def _gemm_runner(shape: dict, cfg: dict, device: torch.device) -> Callable[[], None]:
    from .ops import native_ops as no
    m, n, k = shape["m"], shape["n"], shape["k"]
    a = torch.randn((k, m) if shape["a_mn"] else (m, k), device=device).to(torch.bfloat16)
    b = torch.randn((k, n) if shape["b_mn"] else (n, k), device=device).to(torch.bfloat16)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=device)
    # explicit arguments bypass the table, so a candidate is measured as given
    kw = dict(a_mn=shape["a_mn"], b_mn=shape["b_mn"], out=out, bm=cfg.get("bm", 0), bn=cfg.get("bn", 0),
              two_cta=cfg.get("two_cta", False), max_ctas=cfg.get("max_ctas", 0))
    return lambda: no.gemm(a, b, **kw)


def _conv_runner(shape: dict, cfg: dict, device: torch.device) -> Callable[[], None]:
    from .ops import native_ops as no
    x = torch.randn(shape["batch"], shape["in_h"], shape["in_w"], shape["c"], device=device).to(torch.bfloat16)
    taps = [tuple(t) for t in shape["taps"]]
    wmat = (torch.randn(shape["n_out"], len(taps) * shape["c"], device=device) * 0.05).to(torch.bfloat16)
    out = torch.empty(shape["batch"], shape["out_hw"][0], shape["out_hw"][1], shape["n_out"], dtype=torch.bfloat16,
                      device=device)
    kw = dict(grid_hw=tuple(shape["grid_hw"]), in_mul=shape["in_mul"], taps=taps, out_mul=shape["out_mul"],
              out_off=tuple(shape["out_off"]), bn=cfg.get("bn", 0), tile_rows=cfg.get("tile_rows", 0),
              two_cta=cfg.get("two_cta", False))
    return lambda: no.conv_pass(x, wmat, shape["n_out"], out, **kw)


def tune(shapes: Dict[str, dict], device: torch.device, warmup: int = 2, iters: int = 5,
         log: Optional[Callable[[str], None]] = None) -> dict:
    """Times every candidate of every shape; returns the document to write."""
    from .ops import native as nv
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    entries = {}
    for key, shape in sorted(shapes.items()):
        is_gemm = key.startswith("gemm ")
        candidates = tuning.gemm_candidates(shape["m"], shape["n"]) if is_gemm else tuning.conv_candidates(shape["n_out"])
        results: List[dict] = []
        for cfg in candidates:
            try:
                run = (_gemm_runner if is_gemm else _conv_runner)(shape, cfg, device)
                ms = _time_ms(run, flush, warmup, iters)
                nv.check_status(device)
            except (RuntimeError, ValueError) as e:     # the launcher refused this configuration for this shape
                if log:
                    log(f"{key}: {cfg} skipped ({e})")
                continue
            results.append({"config": cfg, "ms": ms})
        if not results:
            continue
        results.sort(key=lambda r: r["ms"])
        entries[key] = {"best": results[0]["config"], "ms": results[0]["ms"], "candidates": results}
        if log:
            log(f"{key}: best {results[0]['config']} {results[0]['ms']:.4f} ms of {len(results)} candidates")
    return {"device": torch.cuda.get_device_name(device), "entries": entries}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="fbamtrain-autotune")
    ap.add_argument("--model", default="fbam_small", help="preset whose training step supplies the shapes")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--shapes", default=None, help="JSON file {key: geometry} to tune instead of a model's step")
    ap.add_argument("--dump-shapes", default=None, help="write the collected {key: geometry} here")
    ap.add_argument("--out", default="tuning.json")
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        sys.stderr.write("autotune measures on a GPU; none is visible\n")
        return 2
    device = torch.device("cuda", 0)
    if a.shapes:
        with open(a.shapes) as f:
            shapes = json.load(f)
    else:
        shapes = collect_shapes(a.model, a.micro_batch, a.seq, device)
    if a.dump_shapes:
        with open(a.dump_shapes, "w") as f:
            json.dump(shapes, f, indent=1)
    doc = tune(shapes, device, a.warmup, a.iters, log=lambda s: sys.stdout.write(s + "\n"))
    tuning.parse(doc)                                   # what is written must load
    with open(a.out, "w") as f:
        json.dump(doc, f, indent=1)
    sys.stdout.write(f"wrote {a.out}: {len(doc['entries'])} shapes\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
