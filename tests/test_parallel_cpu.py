"""Data-parallel plumbing, rendezvous and the collective wrapper on CPU ranks (gloo, world size 2)."""
import os
import socket
import threading

import pytest
import torch
import torch.multiprocessing as mp

from fbamtrain_b200 import RunConfiguration, Trainer, presets
from fbamtrain_b200.data import SyntheticBatchSource


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg(total=4, micro=2, opt="adamw"):
    d = presets.tiny()
    d["total_batch_size"], d["micro_batch_size"] = total, micro
    d["optimizer"]["type"] = opt
    return RunConfiguration.from_json(d)


def _batches(cfg, n, batch):
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=5, pin=False)
    return [src.next_batch(batch, cfg.train_sequence_length) for _ in range(n)]


def _dp_worker(rank, world, port, mode, opt, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fbamtrain_b200.parallel.dp import DataParallel
    cfg = _cfg(opt=opt)
    tr = Trainer(cfg, device=torch.device("cpu"), dp=DataParallel(mode=mode))
    assert tr.grad_accum_steps == 1
    batches = _batches(cfg, 3, 4)
    losses = []
    for cells, tg in batches:
        lo = rank * 2
        losses.append(float(tr.train_step(cells[lo:lo + 2], tg[lo:lo + 2])))
    tr.dp.gather_optimizer_state(tr)
    state = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    for name, opt_ in tr.optimizers.items():
        for k, v in opt_.state_tensors().items():
            state["opt:" + k] = v.detach().clone()
    torch.save({"params": state, "losses": losses}, os.path.join(out_dir, f"{mode}_{rank}.pt"))
    tr.close()
    dist.destroy_process_group()


def _run(mode, opt, tmp_path, world=2):
    port = _free_port()
    mp.spawn(_dp_worker, args=(world, port, mode, opt, str(tmp_path)), nprocs=world, join=True)
    return [torch.load(os.path.join(tmp_path, f"{mode}_{r}.pt")) for r in range(world)]


def test_dp_allreduce_and_zero1_match_single_process(tmp_path):
    ar = _run("allreduce", "adamw", tmp_path)
    z1 = _run("zero1", "adamw", tmp_path)
    # ranks agree with one another
    for res in (ar, z1):
        for k, v in res[0]["params"].items():
            assert torch.equal(v, res[1]["params"][k]), k
    # sharded optimizer == replicated optimizer (to rounding: CPU backward kernels are not run-to-run exact)
    for k, v in ar[0]["params"].items():
        if "qkv.bias" in k:   # the key bias has a zero gradient in exact arithmetic; Adam amplifies its rounding noise
            continue
        assert torch.allclose(v.float(), z1[0]["params"][k].float(), atol=1e-6), k
    # and both equal one process training on the whole batch with two accumulation steps
    cfg = _cfg()
    tr = Trainer(cfg, device=torch.device("cpu"))
    assert tr.grad_accum_steps == 2
    for cells, tg in _batches(cfg, 3, 4):
        tr.train_step(cells, tg)
    for n, p in tr.model.named_parameters():
        if "qkv.bias" in n:
            continue
        assert torch.allclose(p, ar[0]["params"][n], atol=2e-6), n
    tr.close()
    # loss reported per rank is that rank's share of the global mean
    single = ar[0]["losses"][0] + ar[1]["losses"][0]
    assert single > 0


def test_dp_muon_replicated_matrices_sharded_adam(tmp_path):
    res = _run("zero1", "muon", tmp_path)
    for k, v in res[0]["params"].items():
        assert torch.equal(v, res[1]["params"][k]), k


def _rdv_worker(rank, world, port, q):
    from fbamtrain_b200.parallel import ccl, rendezvous
    comm = rendezvous.perform_ccl_rendezvous("127.0.0.1", port, rank, world, torch.device("cpu"), timeout_s=30)
    ccl.barrier(comm)
    t = torch.full((4,), float(rank + 1))
    ccl.all_reduce_async(comm, t).wait()
    out = torch.zeros(world * 2)
    ccl.all_gather_async(comm, out, torch.full((2,), float(rank))).wait()
    if rank == 0:
        ccl.send_string(comm, "héllo from 0", 1)
        msg = ""
    else:
        msg = ccl.recv_string(comm, 0)
    b = torch.arange(3.0) if rank == 0 else torch.zeros(3)
    ccl.broadcast_async(comm, b, 0).wait()
    sub = ccl.create_subset_communicator(comm, [0])
    q.put((rank, t.tolist(), out.tolist(), msg, b.tolist(), sub is not None))
    rendezvous.teardown(comm)


def test_rendezvous_and_ccl_ops():
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rdv_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert got[0][1] == [3.0] * 4 and got[1][1] == [3.0] * 4
    assert got[0][2] == [0.0, 0.0, 1.0, 1.0]
    assert got[1][3] == "héllo from 0"
    assert got[1][4] == [0.0, 1.0, 2.0]
    assert got[0][5] is True and got[1][5] is False


def test_rendezvous_rejects_bad_ranks():
    from fbamtrain_b200.parallel import rendezvous as rdv
    port = _free_port()
    blob = b"x" * rdv.BLOB_BYTES
    err = {}

    def serve():
        try:
            rdv.serve_blob("127.0.0.1", port, 3, blob, timeout_s=10)
        except rdv.RendezvousError as ex:
            err["e"] = str(ex)

    th = threading.Thread(target=serve)
    th.start()
    with pytest.raises(rdv.RendezvousError):
        rdv.fetch_blob("127.0.0.1", port, 7, timeout_s=5)   # out of range: server closes without a blob
    th.join(20)
    assert "out of range" in err["e"]
    with pytest.raises(rdv.RendezvousError):
        rdv.perform_ccl_rendezvous("127.0.0.1", port, 5, 2, torch.device("cpu"))


def _recover_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fbamtrain_b200.parallel.dp import recover_sharded_state
    n, old_world = 12, 3
    # old world of three; old rank 1 is gone; new rank 0 was old rank 0, new rank 1 was old rank 2, new rank 2 is new
    old = {0: (0, old_world), 1: (2, old_world), 2: None}[rank]
    moment = torch.full((n,), -1.0)
    master = torch.full((n,), -1.0)
    if old is not None:
        per = n // old_world
        moment[old[0] * per:(old[0] + 1) * per] = 10.0 + old[0]
        master[old[0] * per:(old[0] + 1) * per] = 20.0 + old[0]
    params = torch.arange(n, dtype=torch.float32)
    lost = recover_sharded_state([(moment, None), (master, params)], old, None)
    q.put((rank, lost, moment.tolist(), master.tolist()))
    dist.destroy_process_group()


def test_recover_sharded_state_after_membership_change():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_recover_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(3)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    want_moment = [10.0] * 4 + [0.0] * 4 + [12.0] * 4          # the lost slice restarts from zero
    want_master = [20.0] * 4 + [4.0, 5.0, 6.0, 7.0] + [22.0] * 4   # ... and takes its masters from the parameters
    for rank, lost, moment, master in got:
        assert lost == 1 and moment == want_moment and master == want_master, (rank, moment, master)


def _write_recordings(root):
    import numpy as np
    from fbamtrain_b200.data import ArrayRecording, SyntheticRecording
    from fbamtrain_b200.tokenizer import Tokenizer
    os.makedirs(os.path.join(root, "rec"), exist_ok=True)
    for i in range(3):
        r = SyntheticRecording(8, 16, 60, seed=i)
        cells = np.stack([r.frame(t)[0] for t in range(60)])
        ArrayRecording(cells, [r.frame(t)[1] for t in range(60)]).save(os.path.join(root, "rec", f"r{i}.fbrec.npz"))
    Tokenizer(list("abcdefghijklmnopqrstuvwxyz") + ["ab", "th"]).save(os.path.join(root, "tok.txt"))


def _recordings_cfg(micro, total):
    d = presets.tiny()
    d["total_batch_size"], d["micro_batch_size"] = total, micro
    d["tokenizer_file_path"] = "tok.txt"
    d["train_data_config"]["recordings_directory_path"] = "rec"
    d["model_config"]["action_vocab"] = 0
    d["checkpointing"] = {"checkpoint_interval": 2, "checkpoint_directory": "ck", "resume_behavior": "load_latest"}
    return RunConfiguration.from_json(d)


def _dp_loop_worker(rank, world, port, root, q):
    """ZeRO-1 ranks through the whole outer loop on recordings: 3 steps (checkpoint after step 2, which gathers the
    sharded optimizer state collectively), then a fresh trainer resumes from it and repeats step 3."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fbamtrain_b200.parallel.dp import DataParallel
    from fbamtrain_b200.train import run_training
    cfg = _recordings_cfg(micro=2, total=4)
    tr = Trainer(cfg, device=torch.device("cpu"), dp=DataParallel(mode="zero1"), working_dir=root)
    first = [h["loss/train"] for h in run_training(tr, max_steps=3)]
    tr.close()
    dist.barrier()
    tr = Trainer(cfg, device=torch.device("cpu"), dp=DataParallel(mode="zero1"), working_dir=root)
    again = [h["loss/train"] for h in run_training(tr, max_steps=1)]
    tr.close()
    q.put((rank, first, again))
    dist.destroy_process_group()


def test_dp_outer_loop_on_recordings_matches_single_process_and_resumes(tmp_path):
    """Two data-parallel ranks draw the same global batches as one process with gradient accumulation (one seeded
    iterator, per-rank shares), so the loss curves agree; checkpointing inside the loop is collective; the resumed
    ranks repeat the step after the checkpoint."""
    from fbamtrain_b200.train import run_training
    root = str(tmp_path)
    _write_recordings(root)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dp_loop_worker, args=(r, 2, port, root, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict((r, (a, b)) for r, a, b in (q.get(timeout=300) for _ in range(2)))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    single_root = str(tmp_path / "single")
    _write_recordings(single_root)
    tr = Trainer(_recordings_cfg(micro=2, total=4), device=torch.device("cpu"), working_dir=single_root)
    single = [h["loss/train"] for h in run_training(tr, max_steps=3)]
    tr.close()
    # each rank logs its share of the global mean: the shares add up to the single-process loss
    summed = [results[0][0][i] + results[1][0][i] for i in range(3)]
    assert summed == pytest.approx(single, rel=2e-4)
    for r in range(2):
        assert results[r][1][0] == pytest.approx(results[r][0][2], rel=1e-5)   # step 3 repeated after the resume
    # the checkpoint written by two ZeRO-1 ranks resumes in ONE process (state is stored per parameter, the data
    # order does not depend on the number of ranks): it repeats step 3 with the whole batch
    tr = Trainer(_recordings_cfg(micro=2, total=4), device=torch.device("cpu"), working_dir=root)
    alone = [h["loss/train"] for h in run_training(tr, max_steps=1)]
    tr.close()
    assert alone[0] == pytest.approx(results[0][0][2] + results[1][0][2], rel=2e-4)
