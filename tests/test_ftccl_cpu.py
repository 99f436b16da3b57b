"""Fault-tolerant membership on CPU ranks: admission, eviction after a silent failure, catch-up of a late joiner
through shared-state synchronisation, retrying all-reduce.  All failures are injected on the host."""
import time

import pytest
import torch
import torch.multiprocessing as mp

from fbamtrain_b200.parallel.ftccl import (Attribute, FtPeer, MembershipMaster, NativeMembershipMaster, Result,
                                            SharedStateSyncStrategy, TensorInfo, tensor_hash)

MASTERS = {"python": MembershipMaster, "native": NativeMembershipMaster}


def _peer_main(idx, port, q, script):
    torch.manual_seed(idx)
    peer = FtPeer("127.0.0.1", port, torch.device("cpu"), heartbeat_interval_s=0.1, collective_timeout_s=20.0)
    assert peer.connect() == Result.SUCCESS
    try:
        script(idx, peer, q)
    finally:
        if peer.alive:
            peer.leave()


def _script_basic(idx, peer, q):
    assert peer.update_topology(min_world=3, timeout_s=60) == Result.SUCCESS
    assert peer.get_attribute(Attribute.GLOBAL_WORLD_SIZE) == 3
    assert peer.optimize_topology() == Result.SUCCESS
    # shared state: rank with revision 5 wins, others adopt it
    state = torch.full((16,), float(peer.rank))
    rev = 5 if peer.rank == 1 else 3
    res, info = peer.synchronize_shared_state(rev, [TensorInfo("w", state)])
    assert res == Result.SUCCESS and info.revision == 5
    t = torch.full((8,), float(peer.rank + 1))
    res, rinfo = peer.all_reduce(t)
    assert res == Result.SUCCESS
    # the lossy 8-bit variants agree with the exact sum to within the code resolution and move a quarter of the bytes
    from fbamtrain_b200.parallel.ftccl import QuantizationAlgorithm
    gen = torch.Generator().manual_seed(100 + peer.rank)
    mine = torch.randn(1024, generator=gen)
    exact = sum(torch.randn(1024, generator=torch.Generator().manual_seed(100 + r)) for r in range(3))
    for algo in (QuantizationAlgorithm.MIN_MAX, QuantizationAlgorithm.ZERO_POINT_SCALE):
        q_t = mine.clone()
        res, qinfo = peer.all_reduce(q_t, quantization=algo)
        assert res == Result.SUCCESS
        assert float((q_t - exact).abs().max()) < 3 * 8.0 / 255.0      # three peers, range below 8, half a code each
        assert qinfo.tx_bytes < 1024 * 4 * 2 * 2 // 3 // 2
    q.put(("basic", idx, peer.rank, state.tolist()[0], t.tolist()[0], info.rx_bytes, info.tx_bytes))


@pytest.mark.parametrize("kind", ["python", "native"])
def test_admission_shared_state_and_allreduce(kind):
    master = MASTERS[kind](heartbeat_timeout_s=2.0).start()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_peer_main, args=(i, master.port, q, _script_basic)) for i in range(3)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(3)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    master.interrupt()
    assert sorted(g[2] for g in got) == [0, 1, 2]
    assert all(g[3] == 1.0 for g in got)            # everyone holds rank 1's content (highest revision)
    assert all(g[4] == 6.0 for g in got)            # 1 + 2 + 3
    assert sum(1 for g in got if g[5] > 0) == 2     # two receivers
    assert sum(1 for g in got if g[6] > 0) == 1     # one donor


def _script_churn(idx, peer, q):
    """Three peers train a toy quadratic with summed gradients.  Peer 2 fails silently after step 2; the
    survivors notice on the host, re-rendezvous and go on; peer 3 joins later and catches up."""
    late = idx == 3
    w = torch.zeros(4) if not late else torch.full((4,), -99.0)
    step = 0
    if late:
        time.sleep(1.5)
    assert peer.update_topology(min_world=2 if late else 3, timeout_s=60) == Result.SUCCESS
    res, info = peer.synchronize_shared_state(step, [TensorInfo("w", w)], SharedStateSyncStrategy.ENFORCE_POPULAR
                                              if not late else SharedStateSyncStrategy.RECEIVE_ONLY)
    assert res == Result.SUCCESS
    step = info.revision
    target = torch.arange(4.0)
    dropped = 0
    while step < 12:
        if idx == 2 and step == 2:
            peer.inject_failure()          # falls silent between steps; nothing on a device is touched
            q.put(("died", idx, step))
            return
        if peer.membership_changed() or peer.are_peers_pending():
            assert peer.update_topology(min_world=2, timeout_s=60) == Result.SUCCESS
            res, info = peer.synchronize_shared_state(step, [TensorInfo("w", w)])
            assert res == Result.SUCCESS
            step = info.revision
        grad = (w - target) / 3.0
        res, _ = peer.all_reduce_multiple_with_retry([grad], [step], min_world=2)
        if res != Result.SUCCESS:
            dropped += 1                  # drop the step: no update, re-sync at the old revision
            peer.synchronize_shared_state(step, [TensorInfo("w", w)])
            continue
        w -= 0.5 * grad * (3.0 / peer.world_size)   # keep the mean-gradient scale when the world shrinks
        step += 1
        time.sleep(0.15)
    q.put(("done", idx, step, w.tolist(), dropped, peer.world_size))


@pytest.mark.parametrize("kind", ["python", "native"])
def test_silent_failure_eviction_and_late_joiner_catch_up(kind):
    master = MASTERS[kind](heartbeat_timeout_s=0.6).start()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_peer_main, args=(i, master.port, q, _script_churn)) for i in range(4)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(4)]
    for p in procs:
        p.join(60)
    master.interrupt()
    died = [r for r in results if r[0] == "died"]
    done = sorted((r for r in results if r[0] == "done"), key=lambda r: r[1])
    assert len(died) == 1 and died[0][1] == 2
    assert [r[1] for r in done] == [0, 1, 3]
    # survivors and the late joiner end on the same step with identical weights, close to the optimum
    assert all(r[2] == 12 for r in done)
    for r in done[1:]:
        assert r[3] == pytest.approx(done[0][3], abs=1e-6)
    assert done[0][3] == pytest.approx([0.0, 1.0, 2.0, 3.0], abs=0.2)
    assert done[0][5] == 3                     # world grew back to three


def test_tensor_hash_is_content_based():
    a = torch.arange(10.0)
    assert tensor_hash(a) == tensor_hash(a.clone())
    assert tensor_hash(a) != tensor_hash(a + 1)
