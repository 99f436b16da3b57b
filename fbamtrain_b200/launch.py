"""Single-machine launcher: starts one trainer process per rank (and the membership master when the parallel
configuration uses the fault-tolerant transport), prefixes their output with the rank and returns the first
non-zero exit code.

    python -m fbamtrain_b200.launch --nproc 8 -- -c run.json --parallel-config configs/parallel/dp_ccl_fused.json
    python -m fbamtrain_b200.launch --nproc 8 --pipelines 1 -- -c run.json --parallel-config \
        configs/parallel/frame_head_parallel.json
    python -m fbamtrain_b200.launch --nproc 8 --pipelines 2 -- -c run.json --parallel-config \
        configs/parallel/pipelines_ftccl.json        # two pipelines under the membership master

When a rank fails, the others get ``--grace`` seconds to finish and are then stopped (ranks of a fault-tolerant job
carry on instead).  Everything after ``--`` goes to ``fbamtrain_b200.cli`` unchanged; the launcher adds ``--worker_id``, ``--world-size`` /
``--ddp-world-size`` and, for pipelines, ``--master`` on each pipeline's first action-model rank — what the
reference's launcher script does for its binary (reference: ``scripts/run_frame_head_parallel.sh:1-112``).
"""
from __future__ import annotations

import argparse
import subprocess
import sys
import threading
import time
from typing import List

from .config import ParallelConfiguration


def _pump(proc: subprocess.Popen, tag: str) -> None:
    for line in proc.stdout:
        sys.stdout.write(f"[{tag}] {line}")
        sys.stdout.flush()


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--" not in argv:
        raise SystemExit("usage: python -m fbamtrain_b200.launch --nproc N [--pipelines P] -- <cli arguments>")
    split = argv.index("--")
    ap = argparse.ArgumentParser(prog="fbamtrain-launch")
    ap.add_argument("--nproc", type=int, required=True, help="trainer processes (= GPUs) to start")
    ap.add_argument("--pipelines", type=int, default=1,
                    help="with a frame_head_parallel configuration: pipelines running side by side")
    ap.add_argument("--grace", type=float, default=15.0,
                    help="seconds the remaining ranks get to finish after one rank has failed")
    a = ap.parse_args(argv[:split])
    cli_args: List[str] = argv[split + 1:]
    par = None
    if "--parallel-config" in cli_args:
        par = ParallelConfiguration.from_json_file(cli_args[cli_args.index("--parallel-config") + 1])
    procs, threads = [], []

    def start(extra: List[str], tag: str) -> None:
        p = subprocess.Popen([sys.executable, "-m", "fbamtrain_b200.cli"] + cli_args + extra, stdout=subprocess.PIPE,
                             stderr=subprocess.STDOUT, text=True)
        t = threading.Thread(target=_pump, args=(p, tag), daemon=True)
        t.start()
        procs.append(p)
        threads.append(t)

    master = None
    pipeline = par is not None and par.frame_head_parallel.use_frame_head_parallel
    if par is not None and par.ddp_parallel.use_ddp_parallel and par.ddp_parallel.transport == "ftccl":
        master = subprocess.Popen([sys.executable, "-m", "fbamtrain_b200.cli", "--parallel-config",
                                   cli_args[cli_args.index("--parallel-config") + 1], "--ftccl-master"])
        time.sleep(0.5)
    if pipeline:
        if a.nproc % a.pipelines or (a.nproc // a.pipelines) % 2:
            raise SystemExit("--nproc must split into --pipelines pipelines with an even number of ranks each")
        per = a.nproc // a.pipelines
        for r in range(a.nproc):
            if master is not None:
                # pipelines with dynamic membership: every pipeline is a job of its own (its ranks count from 0 and
                # rendezvous at the configured port + the pipeline's number); one GPU per process unless told otherwise
                extra = ["--worker_id", str(r % per), "--replica-id", str(r // per), "--world-size", str(per),
                         "--ddp-world-size", str(a.pipelines)]
                if "--device" not in cli_args:
                    import torch
                    if torch.cuda.is_available():
                        extra += ["--device", f"cuda:{r % torch.cuda.device_count()}"]
                tag = f"pipeline {r // per} rank {r % per}"
            else:
                extra = ["--worker_id", str(r), "--world-size", str(per), "--ddp-world-size", str(a.pipelines)]
                tag = f"rank {r}"
            if r % per == per // 2:
                extra.append("--master")
            start(extra, tag)
    else:
        for r in range(a.nproc):
            start(["--worker_id", str(r), "--ddp-world-size", str(a.nproc)], f"rank {r}")
    # Wait for all ranks; when one fails, the others (which would wait for it in their next collective) are stopped
    # after a short grace period instead of being left hanging.
    code = 0
    while any(p.poll() is None for p in procs):
        failed = [p.returncode for p in procs if p.poll() is not None and p.returncode != 0]
        if failed and master is None:        # (fault-tolerant ranks carry on without the one that failed)
            code = failed[0]
            deadline = time.time() + a.grace
            while time.time() < deadline and any(p.poll() is None for p in procs):
                time.sleep(0.2)
            for p in procs:
                if p.poll() is None:
                    p.terminate()
            for p in procs:
                try:
                    p.wait(10)
                except subprocess.TimeoutExpired:
                    p.kill()
            break
        time.sleep(0.2)
    for p in procs:
        rc = p.wait()
        code = code or rc
    for t in threads:
        t.join(5)
    if master is not None:
        master.terminate()
        master.wait(10)
    return code


if __name__ == "__main__":
    sys.exit(main())
