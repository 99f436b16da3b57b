"""Runs a training command and forwards its JSON metric lines to Weights & Biases.

Lines of the child's stdout that parse as JSON objects containing ``"step"`` are logged with that step (every
other line is passed through), which is the contract of the reference's wrapper
(reference: ``scripts/wandb_log_wrapper.py:28-122``).  The trainer prints such lines when
``FBAMTRAIN_METRICS_JSON`` is set.  Without the ``wandb`` package (or with ``--dry-run``) the parsed metrics are
collected and printed as a summary instead.

    python -m fbamtrain_b200.wandb_log_wrapper --project fbam -- python -m fbamtrain_b200.cli -c run.json
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from typing import Dict, List, Optional


def parse_metric_line(line: str) -> Optional[Dict]:
    line = line.strip()
    if not (line.startswith("{") and line.endswith("}")):
        return None
    try:
        obj = json.loads(line)
    except json.JSONDecodeError:
        return None
    return obj if isinstance(obj, dict) and "step" in obj else None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--project", default="fbamtrain")
    ap.add_argument("--name", default=None)
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
    if not cmd:
        ap.error("no command given")
    run = None
    if not a.dry_run:
        try:
            import wandb  # type: ignore
            run = wandb.init(project=a.project, name=a.name)
        except Exception:  # noqa: BLE001 - missing package or no network: fall back to a local summary
            run = None
    env = dict(os.environ, FBAMTRAIN_METRICS_JSON="1")
    collected: List[Dict] = []
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    for line in proc.stdout:
        metric = parse_metric_line(line)
        if metric is None:
            sys.stdout.write(line)
            continue
        collected.append(metric)
        if run is not None:
            step = metric.pop("step")
            run.log(metric, step=step)
    rc = proc.wait()
    if run is not None:
        run.finish()
    else:
        print(json.dumps({"metrics_logged": len(collected), "last": collected[-1] if collected else None}))
    return rc


if __name__ == "__main__":
    sys.exit(main())
