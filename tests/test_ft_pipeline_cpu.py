"""Dynamic membership for data parallelism over pipelines on CPU ranks: two one-plus-one pipelines (each a gloo job of
its own) train together; one falls silent between steps and the other goes on alone; a fresh pipeline joins later,
receives parameters and optimizer state for both positions and continues in lock-step."""
import os
import socket
import threading
import time

import pytest
import torch
import torch.multiprocessing as mp

from fbamtrain_b200.parallel.ftccl import create_master


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _config():
    from fbamtrain_b200 import RunConfiguration, presets
    d = presets.tiny()
    d["model_config"].update({"action_heads": 2, "lstm_layers": 1})
    d["micro_batch_size"], d["total_batch_size"] = 2, 4
    d["optimizer"]["learning_rate"] = 3e-3
    return RunConfiguration.from_json(d)


def _pipeline_rank(name, rank, static_port, master_port, q, shrunk, total_steps):
    """One rank of pipeline ``name`` ("a" and "b" found the job, "b" dies at step 3, "c" joins after that)."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(static_port)
    dist.init_process_group("gloo", rank=rank, world_size=2)
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.parallel.ft_pipeline import FaultTolerantPipelineReplicas
    from fbamtrain_b200.parallel.pipeline import PipelineTrainer
    cfg = _config()
    late = name == "c"
    if late:
        assert shrunk.wait(240)
    ft = FaultTolerantPipelineReplicas("127.0.0.1", master_port, torch.device("cpu"), expected_replicas=2,
                                       min_replicas=1 if late else 2, late_joiner=late, heartbeat_interval_s=0.1,
                                       collective_timeout_s=20.0)
    tr = PipelineTrainer(cfg, torch.device("cpu"), vocab=32, ft=ft)
    ft.min_replicas = 1
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=5, pin=False)
    cells, targets = src.next_batch(4, cfg.train_sequence_length)
    losses = {}

    def watch():
        while not shrunk.is_set():
            if len(ft.events) > 1 and ft.events[-1]["replicas"] == 1:
                shrunk.set()
            time.sleep(0.05)
    if name == "a" and rank == 0:
        threading.Thread(target=watch, daemon=True).start()

    def finished():
        grown = [e for e in ft.events[(0 if late else 1):] if e["replicas"] == 2]
        if not grown:
            return tr.step_count >= 400
        return tr.step_count >= max(total_steps, grown[0]["step"] + 3)

    while not finished():
        if name == "b" and tr.step_count == 3:
            ft.inject_failure()                      # the whole pipeline falls silent between steps
            q.put(("died", name, rank, tr.step_count, None, None))
            return
        before = tr.step_count
        loss = tr.train_step(cells, targets)
        if tr.step_count > before:
            losses[before] = loss
        time.sleep(0.2)
    params = torch.cat([p.detach().reshape(-1) for _, p in tr.named])
    q.put(("done", name, rank, tr.step_count, params,
           {"events": ft.events, "dropped": ft.dropped_steps, "losses": losses, "rx": ft.rx_bytes}))
    ft.leave()
    dist.destroy_process_group()


def _static_two_replicas(rank, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=4)
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.parallel.pipeline import PipelineTrainer
    cfg = _config()
    tr = PipelineTrainer(cfg, torch.device("cpu"), vocab=32, replicas=2)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=5, pin=False)
    cells, targets = src.next_batch(4, cfg.train_sequence_length)
    q.put((rank, [tr.train_step(cells, targets) for _ in range(3)]))
    dist.destroy_process_group()


def test_pipelines_join_and_leave_a_running_job():
    master = create_master(heartbeat_timeout_s=0.8).start()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    shrunk = ctx.Event()
    ports = {name: _free_port() for name in "abc"}
    procs = [ctx.Process(target=_pipeline_rank, args=(name, rank, ports[name], master.port, q, shrunk, 12))
             for name in "abc" for rank in (0, 1)]
    for p in procs:
        p.start()
    results = [q.get(timeout=400) for _ in range(6)]
    for p in procs:
        p.join(60)
    master.interrupt()
    done = {(r[1], r[2]): r for r in results if r[0] == "done"}
    assert sorted(done) == [("a", 0), ("a", 1), ("c", 0), ("c", 1)]
    assert len([r for r in results if r[0] == "died"]) == 2
    steps = {r[3] for r in done.values()}
    assert len(steps) == 1 and steps.pop() >= 12                     # everyone stopped at the same step
    for rank in (0, 1):                                              # same parameters in both pipelines, per position
        assert torch.equal(done[("a", rank)][4], done[("c", rank)][4])
    info_a, info_c = done[("a", 0)][5], done[("c", 0)][5]
    assert [e["replicas"] for e in info_a["events"]][:2] == [2, 1] and info_a["events"][-1]["replicas"] == 2
    assert min(info_c["losses"]) >= 3 and info_c["rx"] > 0           # joined mid-run and received the state
    assert done[("c", 1)][5]["rx"] > 0                               # ... in the other position too
    # while both founders were there, the job trained like two pipelines under one launcher
    q2 = ctx.Queue()
    port = _free_port()
    static = [ctx.Process(target=_static_two_replicas, args=(r, port, q2)) for r in range(4)]
    for p in static:
        p.start()
    curves = dict(q2.get(timeout=240) for _ in range(4))
    for p in static:
        p.join(60)
    assert [info_a["losses"][k] for k in range(3)] == pytest.approx(curves[0], abs=2e-5)


def _scoped_rank(rank, world, port, q):
    from fbamtrain_b200.parallel.ftccl import (Result, ScopedGroup, SharedStateSyncStrategy, TensorInfo,
                                               synchronize_shared_state)
    group = ScopedGroup("127.0.0.1", port, host_store=rank == 0, prefix="test/1/0", rank=rank, world_size=world,
                        device=torch.device("cpu"), timeout_s=60.0)
    x = torch.full((1000,), float(rank + 1))
    group.all_reduce(x)
    y = torch.full((10,), float(rank))
    group.broadcast(y, src=world - 1)
    objs = group.all_gather_object({"rank": rank, "pad": "x" * (5 * rank)})
    # shared state: the highest revision wins; among equal revisions the most common content
    t = torch.full((64,), float(rank >= 1))
    res, info = synchronize_shared_state(group, 7 if rank >= 1 else 3, [TensorInfo("t", t)],
                                         SharedStateSyncStrategy.ENFORCE_POPULAR)
    q.put((rank, float(x[0]), float(y[0]), [o["rank"] for o in objs], len(objs[-1]["pad"]), res == Result.SUCCESS,
           info.revision, float(t.mean()), info.rx_bytes))
    group.close()


def test_scoped_group_collectives_and_shared_state_on_gloo():
    """The stand-alone communicator of a pipeline position (no default process group involved): sum, broadcast,
    object exchange, and the shared-state comparison in which the member that is behind receives the others' tensor."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_scoped_rank, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(3))
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    for rank, total, bcast, ranks, pad, ok, revision, mean, rx in results:
        assert total == 6.0 and bcast == 2.0 and ranks == [0, 1, 2] and pad == 10
        assert ok and revision == 7 and mean == 1.0
        assert (rx > 0) == (rank == 0)                  # only the member that was behind received anything


def test_peer_that_makes_no_progress_stops_vouching_for_itself():
    """``progress_deadline_s``: the heartbeat thread of a peer whose training thread is stuck (it does not call
    ``note_progress``) stops after the deadline, and the master evicts the peer like a dead process; a peer that keeps
    reporting progress stays."""
    from fbamtrain_b200.parallel.ftccl import FtPeer, Result
    master = create_master(heartbeat_timeout_s=0.6).start()
    try:
        stuck = FtPeer("127.0.0.1", master.port, torch.device("cpu"), heartbeat_interval_s=0.1,
                       owns_default_group=False, progress_deadline_s=0.5)
        moving = FtPeer("127.0.0.1", master.port, torch.device("cpu"), heartbeat_interval_s=0.1,
                        owns_default_group=False, progress_deadline_s=0.5)
        assert stuck.connect() == Result.SUCCESS and moving.connect() == Result.SUCCESS
        deadline = time.time() + 6.0
        while time.time() < deadline:
            moving.note_progress()
            snap = master.snapshot()
            known = set(snap["accepted"]) | set(snap["pending"])
            if stuck.uid not in known:
                break
            time.sleep(0.1)
        snap = master.snapshot()
        known = set(snap["accepted"]) | set(snap["pending"])
        assert stuck.uid not in known and moving.uid in known
        moving.leave()
    finally:
        master.interrupt()
