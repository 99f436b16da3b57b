"""End-to-end numerics validation: the native-kernel trainer against the PyTorch definitions of the same model.

The reference validates its C++ trainer against its PyTorch twin by running both in validation-dump mode for N
steps and comparing every dumped tensor with ``tenscmp -t 0.3`` (reference: ``scripts/validate_numerics.sh:21,
100-123``; dump contents ``src/main.cpp:3492-3564``).  Here both arms live in one package: the same configuration
is stepped with the native backend and with ``ops.set_backend("torch")``, the dumps (``output, h_n, c_n, loss,
frame_embeddings, logits, grad_*, param_*``) are written as safetensors and compared by the native ``tenscmp``.

    python -m fbamtrain_b200.validate_numerics [--steps 2] [--threshold 0.3] [--preset tiny]
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile

import torch

from . import ops, presets, runtime
from .config import RunConfiguration
from .data import SyntheticBatchSource
from .train import Trainer
from .utils import safetensors_io as st


def run(steps: int, threshold: float, preset: str, device: torch.device, out_dir: str) -> int:
    d = presets.PRESETS[preset]("bf16") if preset == "tiny" else presets.PRESETS[preset]()
    if preset == "tiny":
        d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64], "n_embed": 64})
    cfg = RunConfiguration.from_json(d)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point,
                               cfg.model_config.action_vocab, seed=7, pin=False)
    batches = [src.next_batch(cfg.micro_batch_size, cfg.train_sequence_length) for _ in range(steps)]
    paths = {}
    for backend in ("auto", "torch"):
        ops.set_backend(backend)
        try:
            tr = Trainer(cfg, device=device)
            for i, (cells, targets) in enumerate(batches):
                path = os.path.join(out_dir, f"dump_{backend}_{i}.safetensors")
                st.save_file(tr.validation_dump(cells, targets), path)
                paths.setdefault(i, {})[backend] = path
                tr.train_step(cells, targets)
            tr.close()
        finally:
            ops.set_backend("auto")
    failures = 0
    for i in sorted(paths):
        bad, report = runtime.tenscmp(paths[i]["auto"], paths[i]["torch"], threshold)
        print(f"step {i}: {bad} tensor(s) beyond {threshold}")
        if bad:
            sys.stdout.write(report)
        failures += bad
    return failures


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--threshold", type=float, default=0.3)
    ap.add_argument("--preset", default="tiny", choices=list(presets.PRESETS))
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    with tempfile.TemporaryDirectory() as tmp:
        return 1 if run(a.steps, a.threshold, a.preset, torch.device(a.device), tmp) else 0


if __name__ == "__main__":
    sys.exit(main())
