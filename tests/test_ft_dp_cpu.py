"""Trainer under fault-tolerant data parallelism on CPU ranks: a peer falls silent between steps, the others go
on; a fresh peer joins later, receives parameters + optimizer state and continues in lock-step."""
import threading
import time

import torch
import torch.multiprocessing as mp

from fbamtrain_b200.parallel.ftccl import create_master


def _worker(idx, port, q, total_steps, shrunk):
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.parallel.ft_dp import FaultTolerantDataParallel
    from fbamtrain_b200.parallel.ftccl import FtPeer, Result
    torch.manual_seed(0)
    d = presets.tiny()
    d["micro_batch_size"], d["total_batch_size"] = 1, 3
    d["optimizer"]["learning_rate"] = 1e-3
    cfg = RunConfiguration.from_json(d)
    late = idx == 3
    if late:
        assert shrunk.wait(180)               # join only after the survivors have shrunk to two
    peer = FtPeer("127.0.0.1", port, torch.device("cpu"), heartbeat_interval_s=0.1, collective_timeout_s=20.0)
    assert peer.connect() == Result.SUCCESS
    ft = FaultTolerantDataParallel(peer, expected_world=3, min_world=2 if not late else 2)
    ft.late_joiner = late
    if not late:
        ft.min_world = 3                      # the founding members start together
    tr = Trainer(cfg, device=torch.device("cpu"), dp=ft)
    ft.min_world = 2
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=50 + idx, pin=False)
    losses = {}

    def watch():                              # the survivors wait inside a step for the world to be full again
        while not shrunk.is_set():
            if ft.events and ft.events[-1]["world"] == 2:
                shrunk.set()
            time.sleep(0.05)
    if not late:
        threading.Thread(target=watch, daemon=True).start()

    def finished():
        # everyone stops at the same step: at least `total_steps`, and three steps after the joiner's admission
        grown = [e for e in ft.events[(0 if late else 1):] if e["world"] == 3]
        if not grown:
            return tr.step_count >= 400
        return tr.step_count >= max(total_steps, grown[0]["step"] + 3)

    while not finished():
        if idx == 2 and tr.step_count == 3:
            peer.inject_failure()             # silent failure between steps
            q.put(("died", idx, tr.step_count, None, None))
            tr.close()
            return
        cells, tg = src.next_batch(1, cfg.train_sequence_length)
        step_before = tr.step_count
        loss = float(tr.train_step(cells, tg))
        if tr.step_count > step_before:
            losses[step_before] = loss
        time.sleep(0.2)
    params = torch.cat([p.detach().reshape(-1) for p in tr.model.parameters()])
    q.put(("done", idx, tr.step_count, params, {"events": ft.events, "dropped": ft.dropped_steps,
                                                "first_step": min(losses), "rx": ft.rx_bytes}))
    peer.leave()
    tr.close()


def test_trainer_survives_peer_loss_and_admits_joiner():
    master = create_master(heartbeat_timeout_s=0.8).start()      # the native service when the runtime is built
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    shrunk = ctx.Event()
    procs = [ctx.Process(target=_worker, args=(i, master.port, q, 14, shrunk)) for i in range(4)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(4)]
    for p in procs:
        p.join(60)
    master.interrupt()
    done = sorted((r for r in results if r[0] == "done"), key=lambda r: r[1])
    assert [r[1] for r in done] == [0, 1, 3] and len([r for r in results if r[0] == "died"]) == 1
    assert all(r[2] == done[0][2] >= 14 for r in done)
    for r in done[1:]:                                            # identical parameters everywhere
        assert torch.equal(r[3], done[0][3])
    joiner = done[2][4]
    assert joiner["first_step"] >= 1 and joiner["rx"] > 0         # joined mid-run and received the state
    assert len(done[0][4]["events"]) >= 3                         # start, shrink to two, grow to three
    assert done[0][4]["events"][-1]["world"] == 3


class _FakePeer:
    """Host side of a two-member group in which nothing changes: enough for the step logic around the reduction."""
    world_size, rank, epoch, uid = 2, 0, 1, 1

    def gate(self, step, timeout_s=0.0):
        return True

    def membership_changed(self):
        return False

    def are_peers_pending(self):
        return False


class _HalfAppliedStep:
    """Stands in for the fused reduction when a peer falls silent after the first bucket: the action model's
    optimizer has run (parameters, moments, masters and its step counter moved on), the frame head's has not."""
    rank, world_size, grad_scale = 0, 2, 1.0

    def reduce_and_step(self, trainer):
        opt = trainer.optimizers["action_model"]
        shard = (self.rank, self.world_size)                  # the fused kernels update this member's slice only
        if getattr(opt, "groups", None) is not None:
            opt.step(shard=shard)
        elif hasattr(opt, "muon"):
            opt.step_count += 1
            opt.muon.step()
            opt.adam.step(shard=shard) if opt.adam.groups is not None else opt.adam.step()
        else:
            opt.step()
        return True


def _state_of(trainer):
    out = {"param/" + n: p.detach().clone() for n, p in trainer.model.named_parameters()}
    for scope, opt in trainer.optimizers.items():
        for name, t in opt.state_tensors().items():
            out[scope + "/" + name] = t.detach().clone()
        out[scope + "/step_count"] = torch.tensor(opt.step_count)
    return out


def test_dropped_fused_step_leaves_no_trace(monkeypatch):
    """A fused step that reports an expired device-side wait after part of it was applied is undone as a whole:
    parameters, every optimizer tensor and the step counters equal their values before the step."""
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.parallel.ft_dp import FaultTolerantDataParallel
    torch.manual_seed(0)
    for kind in ("adamw", "muon"):
        d = presets.tiny()
        d["optimizer"]["type"] = kind
        cfg = RunConfiguration.from_json(d)
        tr = Trainer(cfg, device=torch.device("cpu"))
        src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=1, pin=False)
        cells, tg = src.next_batch(cfg.micro_batch_size, cfg.train_sequence_length)
        tr.train_step(cells, tg)                       # one committed step: moments and counters are non-trivial
        tr.zero_grad()
        tr._forward_backward(cells, tg)                # gradients of the step that will be dropped
        before = _state_of(tr)
        ft = FaultTolerantDataParallel(_FakePeer(), expected_world=2, mode="fused")
        ft.inner = _HalfAppliedStep()
        monkeypatch.setattr(ft, "_fused_step_completed", lambda trainer: False)
        monkeypatch.setattr(ft, "_retopologize", lambda trainer, joining=False: True)
        monkeypatch.setattr(ft, "_sync_state", lambda trainer, joining=False: True)
        assert ft.reduce_and_step(tr) is False
        assert ft.dropped_steps == 1
        after = _state_of(tr)
        assert before.keys() == after.keys()
        for k in before:
            assert torch.equal(before[k], after[k]), (kind, k)
        # and the half-applied step really had changed something before the rollback
        ft2 = FaultTolerantDataParallel(_FakePeer(), expected_world=2, mode="fused")
        ft2.inner = _HalfAppliedStep()
        monkeypatch.setattr(ft2, "_fused_step_completed", lambda trainer: True)
        assert ft2.reduce_and_step(tr) is True
        changed = _state_of(tr)
        assert any(not torch.equal(before[k], changed[k]) for k in before if k.startswith("action_model/")), kind
        tr.close()
