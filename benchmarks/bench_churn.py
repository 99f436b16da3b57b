"""Fault-tolerant data-parallel churn run on the GPUs of one machine.

    python benchmarks/bench_churn.py --gpus 4 --leavers 1 --interval 10 --steps 50 [--mode fused|allreduce]
    python benchmarks/bench_churn.py --gpus 4 --no-churn --steps 50 --save curve.json    # uninterrupted, same seeds

One process per GPU plus a membership master in the parent.  The last ``leavers`` ranks leave in an orderly way
BETWEEN steps (nothing of theirs in flight) after ``interval`` committed steps and end; ``interval`` steps later
fresh processes on the same GPUs connect as new peers, are admitted at the next collective phase gate and receive
parameters and optimizer state from a survivor (no checkpoint involved); after another ``interval`` steps they
leave again, and so on.  Every membership change re-initialises the process group and, in the fused mode,
re-allocates the peer-memory windows.

The parent prints one JSON line: steady-state frames/s at full and reduced world (median step time of each phase,
host clock around a synchronised step on rank 0), per membership change the time spent in the phase gate
(re-rendezvous + window rebuild + shared-state sync) and the duration of the whole step that contained it
(recovery: change noticed → next step committed), bytes moved for catch-up, dropped steps, and the loss curve;
``--compare FILE`` adds the largest loss difference to a curve saved by an earlier (uninterrupted) run.

NVLink multicast is kept out of this run (NCCL_NVLS_ENABLE=0, no multicast binding of the peer windows, plain
peer loads/stores in the fused kernels): a rank whose memory is bound to a multicast object must not go away.
Reference protocol: ``src/main.cpp:266-320, 350-478, 3672-3767``; it publishes no recovery-time figure.
"""
from __future__ import annotations

import argparse
import json
import os
import queue
import statistics
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


def _worker(idx, port, a, q, go):
    """``go`` is None for a founding member; a late joiner builds its model and then waits for it."""
    import torch
    cpu = a.device == "cpu"                           # host-logic rehearsal on gloo ranks
    if not cpu:
        torch.cuda.set_device(idx)
    dev = torch.device("cpu") if cpu else torch.device("cuda", idx)
    sync = (lambda: None) if cpu else (lambda: torch.cuda.synchronize(dev))
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.parallel.ft_dp import FaultTolerantDataParallel
    from fbamtrain_b200.parallel.ftccl import FtPeer

    late = go is not None
    torch.manual_seed(0)
    if a.model == "tiny":
        d = presets.tiny()
        d["micro_batch_size"], d["total_batch_size"] = a.micro_batch, a.micro_batch * a.gpus
    else:
        d = presets.PRESETS[a.model](a.micro_batch, a.gpus)
    d["train_sequence_length"] = d["validation_sequence_length"] = a.seq
    d["max_training_steps"] = a.steps
    cfg = RunConfiguration.from_json(d)
    peer = FtPeer("127.0.0.1", port, dev, heartbeat_interval_s=0.1, collective_timeout_s=60.0)
    floor = a.gpus if a.no_churn else a.gpus - a.leavers
    ft = FaultTolerantDataParallel(peer, expected_world=a.gpus, min_world=floor if late else a.gpus, mode=a.mode,
                                   full_world_poll_s=0.05)
    ft.late_joiner = late
    joined_at = [0.0]

    def gate():
        if late:
            q.put(("ready", idx, 0, None))
            go.wait()
        joined_at[0] = time.perf_counter()
    ft.ready_gate = gate
    tr = Trainer(cfg, device=dev, dp=ft)             # attaches: founding members wait for each other here
    join_seconds = time.perf_counter() - joined_at[0]
    ft.min_world = floor
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, tr.vocab,
                               seed=1000 + idx, pin=not cpu)
    is_leaver = idx >= a.gpus - a.leavers and not a.no_churn
    first_step = tr.step_count
    losses, times, worlds = {}, {}, {}
    reduced_since = None
    while tr.step_count < a.steps:
        step = tr.step_count
        if not a.no_churn:
            # `interval` steps at the reduced world, then hold at the phase gate until the replacement is admitted
            if peer.world_size < a.gpus:
                reduced_since = step if reduced_since is None else reduced_since
                ft.wait_for_full_world = step >= reduced_since + a.interval
            else:
                reduced_since, ft.wait_for_full_world = None, False
        if is_leaver and step >= first_step + a.interval and step + a.interval < a.steps:
            sync()
            peer.leave()                              # orderly, between steps
            q.put(("left", idx, step, None))
            tr.close()
            return
        src._calls = step                             # the data of step s is the same whoever computes it
        cells, tg = src.next_batch(a.micro_batch, a.seq)
        sync()
        t0 = time.perf_counter()
        loss = tr.train_step(cells, tg)
        val = float(loss)                             # synchronises
        t1 = time.perf_counter()
        if tr.step_count > step:
            losses[step], times[step], worlds[step] = val, t1 - t0, peer.world_size
            if idx == 0:
                q.put(("progress", 0, tr.step_count, None))
    sync()
    q.put(("done", idx, tr.step_count, {"losses": losses, "times": times, "worlds": worlds, "events": ft.events,
                                        "dropped": ft.dropped_steps, "rx": ft.rx_bytes, "tx": ft.tx_bytes,
                                        "join_seconds": join_seconds if late else None, "first_step": first_step}))
    peer.leave()
    tr.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=4)
    ap.add_argument("--leavers", type=int, default=1)
    ap.add_argument("--interval", type=int, default=10)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--model", default="fbam_small")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--mode", default="fused", choices=["fused", "allreduce"])
    ap.add_argument("--no-churn", action="store_true")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--save", default="")
    ap.add_argument("--compare", default="")
    a = ap.parse_args()

    import torch.multiprocessing as mp
    from fbamtrain_b200.parallel.ftccl import create_master
    master = create_master(heartbeat_timeout_s=15.0).start()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = {i: ctx.Process(target=_worker, args=(i, master.port, a, q, None)) for i in range(a.gpus)}
    for p in procs.values():
        p.start()
    running = set(range(a.gpus))
    progress, report0, joiners = 0, None, []
    waiting = {}                                      # idx -> (go event, step at which to release it, ready?)
    deadline = time.time() + 3000
    t_start = time.time()
    while running and time.time() < deadline:
        try:
            kind, idx, step, payload = q.get(timeout=0.2)
        except queue.Empty:
            kind = None
        if kind is not None and kind != "progress":
            sys.stderr.write(f"[churn] t={time.time() - t_start:6.1f}s {kind} slot={idx} step={step} "
                             f"progress={progress}\n")
        if kind == "progress":
            progress = max(progress, step)
        elif kind == "left":
            procs[idx].join(120)
            running.discard(idx)
            go = ctx.Event()                          # the replacement warms up now and joins `interval` steps later
            waiting[idx] = [go, step + a.interval, False]
            procs[idx] = ctx.Process(target=_worker, args=(idx, master.port, a, q, go))
            procs[idx].start()
            running.add(idx)
        elif kind == "ready":
            waiting[idx][2] = True
        elif kind == "done":
            running.discard(idx)
            if idx == 0:
                report0 = payload
            elif payload.get("join_seconds") is not None:
                joiners.append({"rank_slot": idx, "first_step": payload["first_step"],
                                "join_s": round(payload["join_seconds"], 3), "rx_bytes": payload["rx"]})
            procs[idx].join(120)
        for idx, (go, at_step, ready) in list(waiting.items()):
            if ready and progress >= at_step:
                sys.stderr.write(f"[churn] t={time.time() - t_start:6.1f}s go slot={idx} progress={progress}\n")
                go.set()
                del waiting[idx]
    for go, _, _ in waiting.values():
        go.set()
    master.interrupt()
    if report0 is None:
        raise SystemExit("rank 0 did not report")
    times, losses, worlds = report0["times"], report0["losses"], report0["worlds"]
    per_rank = a.micro_batch * a.seq
    change_steps = {e["step"] for e in report0["events"][1:]}
    steady = {}
    for s, t in times.items():
        if s > 2 and s not in change_steps:
            steady.setdefault(worlds[s], []).append(t)
    out = {
        "bench": "ft_dp_churn", "model": a.model, "n_gpus": a.gpus, "leavers": 0 if a.no_churn else a.leavers,
        "interval_steps": a.interval, "steps": a.steps, "mode": a.mode, "dtype": "bf16",
        "steady_frames_per_s_by_world": {str(w): round(per_rank * w / statistics.median(ts), 1)
                                         for w, ts in sorted(steady.items())},
        "membership_changes": [{"step": e["step"], "world": e["world"], "phase_gate_s": round(e["seconds"], 3),
                                "recovery_s": round(times.get(e["step"], float("nan")), 3)}
                               for e in report0["events"][1:]],
        "joiners": joiners, "dropped_steps": report0["dropped"], "rank0_tx_bytes": report0["tx"],
        "final_loss": losses[max(losses)], "timing": "host clock around a synchronised step on rank 0",
        "data": "synthetic seeded frames/actions, random-init weights",
    }
    curve = [losses[s] for s in sorted(losses)]
    if a.save:
        with open(a.save, "w") as f:
            json.dump({"losses": curve}, f)
    if a.compare and os.path.exists(a.compare):
        with open(a.compare) as f:
            other = json.load(f)["losses"]
        n = min(len(other), len(curve))
        out["max_abs_loss_diff_vs_uninterrupted"] = max(abs(curve[i] - other[i]) for i in range(n))
        out["final_loss_uninterrupted"] = other[n - 1]
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
